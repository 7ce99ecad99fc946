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
// Fused all-gather: a launch may carry `g_ctas` extra trailing CTAs that do no MMA work at all.
// They pull the row shards of the NEXT weight of the layer schedule from the peers' memory over
// NVLink (cp.async.bulk peer -> shared -> local staging buffer, 24 x 8 KB in flight per CTA)
// while the other CTAs run this GEMM from the staging buffer the previous launch filled. Stream
// order is the only synchronisation: no flags, no polling, the MMA pipeline is never throttled.
//
// Fused all-reduce (tensor parallelism): in out_mode 5 every tile is stored into this rank's
// symmetric buffer and counted per 128-row block; trailing reducer CTAs wait (bounded) until a
// block they own is complete on every rank, sum it through NVSwitch (multimem.ld_reduce, or peer
// loads) and write the sum into every rank's buffer (multimem.st, or peer stores) while the other
// CTAs keep computing: reduce-scatter + all-gather inside the GEMM launch.
//
// Large problems run on gemm_bf16_pair_kernel below: one 256x256 tile per 2-CTA cluster with
// tcgen05.mma.cta_group::2 (each CTA stages its 128 rows of A and its half of B; the partner's TMA
// loads credit the leader's mbarrier directly, no multicast loads).
//
// Replaces the cuBLAS calls behind the reference's LoRA kernels (src/axolotl/kernels/lora.py:226-280)
// and, with the prefetch / reducer CTAs, the NCCL all-gather of its FSDP2 units and the
// all-reduce of its tensor-parallel layers.
#include <cstdlib>

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
  int group_m;  // m tiles per rasterisation band (the A rows of a band stay L2 resident)
  int* status;
  // out_mode 3: bf16 reduce-add of every tile into red_mc (an NVSwitch multicast address: the add
  // lands in the buffer of every GPU bound to it = all-reduce inside the epilogue);
  // out_mode 4: same through plain peer atomics into red_ptrs[0..red_world)
  void* red_mc;
  unsigned long long red_ptrs[8];
  int red_world;
  // out_mode 5: two-shot all-reduce fused into the launch. Every tile is stored (bf16) into this
  // rank's symmetric buffer C and counted in cnt[m_blk]; `r_ctas` trailing reducer CTAs wait until a
  // 128-row block they own (m_blk % red_world == red_rank) is complete on EVERY rank, sum it over
  // the ranks (multimem.ld_reduce through the switch, or peer loads) and write the sum into every
  // rank's buffer (multimem.st, or peer stores), while the other CTAs keep computing tiles.
  int r_ctas;
  int red_rank;
  unsigned long long cnt_ptrs[8];  // int32 [num_m] completion counters of every rank
  // prefetch of a row-sharded matrix by the trailing g_ctas CTAs (0 = none)
  int g_ctas;
  int g_world;
  const unsigned long long* g_peer_bases;  // DEVICE array [g_world]: arena address of every rank
  unsigned long long g_shard_offset;       // byte offset of the weight's shard inside an arena
  unsigned long long g_shard_bytes;        // bytes per rank
  unsigned long long g_total_bytes;        // g_world * g_shard_bytes (multiple of 8 KB)
  unsigned char* g_dst;                    // local staging buffer
  // CTA-pair kernel only. epi 1 (GLU forward): B holds gate rows [0, I) and up rows [I, 2I); a
  // cluster's tile is 256 rows x (128 gate + 128 up) columns (rank 0 stages the gate rows, rank 1 the
  // up rows of the same 128 columns), N counts the I columns of h. The epilogue stores gate|up into C
  // ([M, 2I], optional) and h = act(gate) * up into H. epi 2 (GLU backward): the accumulator is dh
  // [M, I]; the epilogue reads gate|up from Cin ([M, 2I]) and stores d_gate | d_up into C ([M, 2I],
  // may alias Cin).
  int epi;
  int glu_kind;     // 0 silu, 1 gelu (tanh)
  float glu_limit;  // > 0: clamped GLU
  void* H;
  long long ldh;
  int epi_sleep_ns;   // back-off of the epilogue warps while they wait for an accumulator (0 = spin)
  int prod_sleep_ns;  // back-off of the TMA producer while it waits for a free stage (0 = spin)
  // bf16 results leave through swizzled shared-memory staging tiles and TMA tile stores (full 128-byte
  // lines, no per-thread row stores); 0 = every thread stores its own row (fp32 output, beta != 0,
  // unaligned C)
  int tma_store;
};

int g_epi_sleep_ns = 64, g_prod_sleep_ns = 0, g_pair_group_m = 0, g_pair_tma_store = 1, g_pair_band_mb = 32;

// Row `lane` of a 32-row staging tile with 128-byte rows (64 bf16) and the 128-byte swizzle the
// tensor map expects: 16-byte chunk j of row r sits at chunk position j ^ (r & 7). The tile base is
// 1024-byte aligned.
__device__ __forceinline__ void stage_row128(uint8_t* tile, int lane, const uint4 (&w)[8]) {
  uint8_t* rowp = tile + lane * 128;
#pragma unroll
  for (int j = 0; j < 8; ++j) *reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4)) = w[j];
}
// Same for 64-byte rows (32 bf16) and the 64-byte swizzle: chunk j of row r sits at j ^ ((r >> 1) & 3).
__device__ __forceinline__ void stage_row64(uint8_t* tile, int lane, const uint4 (&w)[4]) {
  uint8_t* rowp = tile + lane * 64;
#pragma unroll
  for (int j = 0; j < 4; ++j) *reinterpret_cast<uint4*>(rowp + ((j ^ ((lane >> 1) & 3)) << 4)) = w[j];
}
__device__ __forceinline__ uint4 pack8(const uint32_t* r, float alpha) {
  uint4 o;
  o.x = pack_bf16x2(__uint_as_float(r[0]) * alpha, __uint_as_float(r[1]) * alpha);
  o.y = pack_bf16x2(__uint_as_float(r[2]) * alpha, __uint_as_float(r[3]) * alpha);
  o.z = pack_bf16x2(__uint_as_float(r[4]) * alpha, __uint_as_float(r[5]) * alpha);
  o.w = pack_bf16x2(__uint_as_float(r[6]) * alpha, __uint_as_float(r[7]) * alpha);
  return o;
}

// Spin on an mbarrier with a pause between polls: the waiting warps stop competing for issue slots
// (and for the power budget of a kernel that runs against the board limit) with the MMA stream.
__device__ __forceinline__ bool mbar_wait_backoff(uint64_t* bar, uint32_t parity, int* status, int code,
                                                  int sleep_ns) {
  if (mbar_test_wait(bar, parity)) return true;
  if (sleep_ns <= 0) return mbar_wait_spin(bar, parity, status, code);
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_test_wait(bar, parity)) {
    __nanosleep(sleep_ns);
    if ((++spins & 0xFF) == 0 && global_timer_ns() - t0 > AXB_WAIT_BUDGET_NS) {
      if (status) atomicCAS(status, 0, code);
      return false;
    }
  }
  return true;
}

// GLU activations on the special-function units (ex2 / rcp / tanh approximations: a couple of ulp,
// far below the bf16 rounding of the results). glu_act_and_grad returns act(g) and writes act'(g).
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float glu_act(float g, int kind) {
  if (kind == 0) return g * __fdividef(1.f, 1.f + __expf(-g));
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * g * (1.f + tanh_fast(k0 * (g + k1 * g * g * g)));
}
__device__ __forceinline__ float glu_act_and_grad(float g, int kind, float& grad) {
  if (kind == 0) {
    const float s = __fdividef(1.f, 1.f + __expf(-g));
    const float a = g * s;
    grad = s + a * (1.f - s);
    return a;
  }
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float t = tanh_fast(k0 * (g + k1 * g * g * g));
  grad = 0.5f * (1.f + t) + 0.5f * g * (1.f - t * t) * k0 * (1.f + 3.f * k1 * g * g);
  return 0.5f * g * (1.f + t);
}

constexpr int GATHER_CHUNK = 8192;
constexpr int GATHER_SLOTS = 4;   // per warp
constexpr int GATHER_WARPS = 6;   // every warp of a gather CTA drives its own slot ring

// Body of a gather CTA: warp w (lane 0) copies chunks (cta*6 + w) + i * (n_ctas*6) through its
// private ring of 4 x 8 KB shared-memory slots. Loads run 3 chunks ahead of the stores.
__device__ __forceinline__ void gather_cta_body(const GemmParams& p, int gather_cta, int n_ctas,
                                                uint8_t* smem, uint64_t* bars) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp < GATHER_WARPS && lane == 0)
    for (int s = 0; s < GATHER_SLOTS; ++s) mbar_init(&bars[warp * GATHER_SLOTS + s], 1);
  mbar_fence_init();
  __syncthreads();
  if (warp >= GATHER_WARPS || lane != 0) return;
  uint8_t* slots = smem + warp * GATHER_SLOTS * GATHER_CHUNK;
  uint64_t* bar = bars + warp * GATHER_SLOTS;
  const unsigned long long n_chunks = p.g_total_bytes / GATHER_CHUNK;
  const unsigned long long stride = (unsigned long long)n_ctas * GATHER_WARPS;
  const unsigned long long c0 = (unsigned long long)gather_cta * GATHER_WARPS + warp;
  const long long n_mine = c0 < n_chunks ? (long long)((n_chunks - c0 + stride - 1) / stride) : 0;
  auto issue_load = [&](long long i) {
    const unsigned long long byte = (c0 + i * stride) * GATHER_CHUNK;
    const unsigned long long owner = byte / p.g_shard_bytes;
    const unsigned char* src = reinterpret_cast<const unsigned char*>(p.g_peer_bases[owner]) +
                               p.g_shard_offset + (byte - owner * p.g_shard_bytes);
    const int slot = (int)(i % GATHER_SLOTS);
    mbar_expect_tx(&bar[slot], GATHER_CHUNK);
    bulk_load(slots + slot * GATHER_CHUNK, src, GATHER_CHUNK, &bar[slot]);
  };
  long long issued = 0;
  for (; issued < GATHER_SLOTS - 1 && issued < n_mine; ++issued) issue_load(issued);
  for (long long i = 0; i < n_mine; ++i) {
    const int slot = (int)(i % GATHER_SLOTS);
    if (!mbar_wait(&bar[slot], (uint32_t)((i / GATHER_SLOTS) & 1), p.status, AXB_TIMEOUT_PEER_FLAG))
      break;
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(
                     p.g_dst + (c0 + i * stride) * GATHER_CHUNK),
                 "r"(smem_u32(slots + slot * GATHER_CHUNK)), "r"(GATHER_CHUNK)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    if (issued < n_mine) {
      // the slot of chunk `issued` was last read by the store of chunk i-1: all but the newest
      // store group must have finished reading shared memory
      asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      issue_load(issued);
      ++issued;
    }
  }
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

AXB_DEVICE int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Body of a reducer CTA (out_mode 5), see GemmParams. All 192 threads move data; thread 0 polls.
__device__ __forceinline__ void reducer_cta_body(const GemmParams& p, int reducer, int n_reducers, int num_m,
                                                 int target) {
  __shared__ int s_ok;
  const long long vec_per_row = p.N >> 3;  // 16-byte vectors (N % 8 == 0)
  int owned = 0;
  for (int blk = p.red_rank; blk < num_m; blk += p.red_world, ++owned) {
    if (owned % n_reducers != reducer) continue;
    if (threadIdx.x == 0) {
      int ok = 1;
      const unsigned long long t0 = global_timer_ns();
      for (int r = 0; r < p.red_world && ok; ++r) {
        const int* c = reinterpret_cast<const int*>(p.cnt_ptrs[r]) + blk;
        while (ld_acquire_sys(c) < target) {
          if (global_timer_ns() - t0 > AXB_WAIT_BUDGET_NS) {  // report and give up
            atomicExch(p.status, AXB_TIMEOUT_PEER_FLAG);
            ok = 0;
            break;
          }
          __nanosleep(200);
        }
      }
      s_ok = ok;
    }
    __syncthreads();
    if (!s_ok) return;
    const int rows = min(BM, p.M - blk * BM);
    const long long n_vec = rows * vec_per_row;
    if (p.red_mc) {
      // 8 independent in-switch reductions in flight per thread: the round trip through NVSwitch is
      // microseconds, so memory-level parallelism (not instruction rate) sets the bandwidth
      constexpr int U = 8;
      for (long long v0 = threadIdx.x; v0 < n_vec; v0 += (long long)blockDim.x * U) {
        uint32_t q[U][4];
        __nv_bfloat16* addr[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long v = v0 + (long long)u * blockDim.x;
          const long long vv = v < n_vec ? v : v0;
          addr[u] = reinterpret_cast<__nv_bfloat16*>(p.red_mc) + ((long long)blk * BM + vv / vec_per_row) * p.ldc +
                    (vv % vec_per_row) * 8;
          asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                       : "=r"(q[u][0]), "=r"(q[u][1]), "=r"(q[u][2]), "=r"(q[u][3])
                       : "l"(addr[u])
                       : "memory");
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (v0 + (long long)u * blockDim.x < n_vec)
            asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(addr[u]),
                         "r"(q[u][0]), "r"(q[u][1]), "r"(q[u][2]), "r"(q[u][3])
                         : "memory");
        }
      }
    } else {
      constexpr int U = 4;
      for (long long v0 = threadIdx.x; v0 < n_vec; v0 += (long long)blockDim.x * U) {
        uint4 x[U][8];
        long long off[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long v = v0 + (long long)u * blockDim.x;
          const long long vv = v < n_vec ? v : v0;
          off[u] = ((long long)blk * BM + vv / vec_per_row) * p.ldc + (vv % vec_per_row) * 8;
          for (int r = 0; r < p.red_world; ++r)   // peer data was written during this launch: volatile loads
            asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(x[u][r].x), "=r"(x[u][r].y), "=r"(x[u][r].z), "=r"(x[u][r].w)
                         : "l"(reinterpret_cast<const __nv_bfloat16*>(p.red_ptrs[r]) + off[u])
                         : "memory");
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (v0 + (long long)u * blockDim.x >= n_vec) continue;
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          for (int r = 0; r < p.red_world; ++r) {
            const uint32_t w[4] = {x[u][r].x, x[u][r].y, x[u][r].z, x[u][r].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = unpack_bf16x2(w[e]);
              acc[2 * e] += f.x;
              acc[2 * e + 1] += f.y;
            }
          }
          const uint4 o = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                     pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
          for (int r = 0; r < p.red_world; ++r)
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.red_ptrs[r]) + off[u]) = o;
        }
      }
    }
    __syncthreads();
    // the block is reduced: re-arm its counter on every rank for the next launch (launches are
    // separated by a cross-rank barrier, so nobody counts into it before this store)
    if (threadIdx.x < p.red_world) reinterpret_cast<int*>(p.cnt_ptrs[threadIdx.x])[blk] = 0;
  }
}

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
};

__device__ __forceinline__ void decode_tile(int tile, int num_m, int num_n, int splits, int& m_blk,
                                            int& n_blk, int& split, int GROUP_M) {
  split = tile % splits;
  tile /= splits;
  const int per_group = GROUP_M * num_n;
  const int group = tile / per_group;
  const int first_m = group * GROUP_M;
  const int gsz = min(num_m - first_m, GROUP_M);
  const int in_group = tile - group * per_group;
  m_blk = first_m + in_group % gsz;
  n_blk = in_group / gsz;
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA,
                             const __grid_constant__ CUtensorMap tmB,
                             const __grid_constant__ CUtensorMap tmA2,
                             const __grid_constant__ CUtensorMap tmB2, const GemmParams p) {
  using C = Cfg<BN>;
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

  const int n_workers = (int)gridDim.x - p.g_ctas - p.r_ctas;  // CTAs that run GEMM tiles
  if ((int)blockIdx.x >= n_workers + p.g_ctas) {
    reducer_cta_body(p, (int)blockIdx.x - n_workers - p.g_ctas, p.r_ctas, (p.M + BM - 1) / BM,
                     4 * ((p.N + BN - 1) / BN));
    return;
  }
  if ((int)blockIdx.x >= n_workers) {
    gather_cta_body(p, (int)blockIdx.x - n_workers, p.g_ctas, smem, bars);
    return;
  }

  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int nk_main = (p.K + BK - 1) / BK;
  const int nk_ext = (p.K2 + BK - 1) / BK;
  const int nk_total = nk_main + nk_ext;
  const int total_tiles = num_m * num_n * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
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
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += n_workers) {
        int m_blk, n_blk, split;
        decode_tile(tile, num_m, num_n, p.splits, m_blk, n_blk, split, p.group_m);
        const int kb0 = (int)((long long)nk_total * split / p.splits);
        const int kb1 = (int)((long long)nk_total * (split + 1) / p.splits);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, AXB_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&full_bar[stage], C::STAGE_BYTES);
          const bool ext = kb >= nk_main;
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
          if (++stage == C::STAGES) {
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
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += n_workers, ++it) {
        int m_blk, n_blk, split;
        decode_tile(tile, num_m, num_n, p.splits, m_blk, n_blk, split, p.group_m);
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
    // ------------------------------------------------------------ epilogue warps
    const int lane_group = warp & 3;  // TMEM lanes [32*lane_group, 32*lane_group+32)
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += n_workers, ++it) {
      int m_blk, n_blk, split;
      decode_tile(tile, num_m, num_n, p.splits, m_blk, n_blk, split, p.group_m);
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
        if (p.out_mode == 0 || p.out_mode == 5) {
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
        } else if (p.out_mode == 3 || p.out_mode == 4) {
          // all-reduce fused into the epilogue (requires N % 8 == 0 and ldc % 8 == 0)
          const long long off = row * p.ldc + col0;
          const int nvec = full_chunk ? 4 : ((p.N - col0) >> 3);
          for (int q = 0; q < nvec; ++q) {
            const uint32_t w0 = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
            const uint32_t w1 = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
            const uint32_t w2 = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
            const uint32_t w3 = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
            if (p.out_mode == 3) {
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.red_mc) + off + q * 8;
              asm volatile("multimem.red.relaxed.sys.global.add.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(dst),
                           "r"(w0), "r"(w1), "r"(w2), "r"(w3)
                           : "memory");
            } else {
              for (int r2 = 0; r2 < p.red_world; ++r2) {
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.red_ptrs[r2]) + off + q * 8;
                asm volatile("red.relaxed.sys.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(dst),
                             "r"(w0), "r"(w1), "r"(w2), "r"(w3)
                             : "memory");
              }
            }
          }
        } else {
          float* crow = reinterpret_cast<float*>(p.C) + row * p.ldc + col0;
          for (int j = 0; j < 32 && col0 + j < p.N; ++j) atomicAdd(crow + j, v[j]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&tempty_bar[acc]);
        if (p.out_mode == 5) {
          // this warp's quarter of the tile is stored: publish it (release at system scope covers the
          // other lanes' stores, ordered before this point by the warp barrier)
          int* c = reinterpret_cast<int*>(p.cnt_ptrs[p.red_rank]) + m_blk;
          asm volatile("red.release.sys.global.add.s32 [%0], 1;" ::"l"(c) : "memory");
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

template <int BN, bool A_MN, bool B_MN>
int launch_gemm(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tA2,
                const CUtensorMap& tB2, const GemmParams& p, int sm_count, cudaStream_t stream) {
  using C = Cfg<BN>;
  auto kern = gemm_bf16_tcgen05_kernel<BN, A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int tiles = num_m * num_n * p.splits;
  int workers = sm_count - p.g_ctas - p.r_ctas;
  if (tiles < workers) workers = tiles;
  const int grid = workers + p.g_ctas + p.r_ctas;
  kern<<<grid, kThreads, C::SMEM_BYTES, stream>>>(tA, tB, tA2, tB2, p);
  return (int)cudaGetLastError();
}

template <int BN>
int dispatch_major(int a_mn, int b_mn, const CUtensorMap& tA, const CUtensorMap& tB,
                   const CUtensorMap& tA2, const CUtensorMap& tB2, const GemmParams& p,
                   int sm_count, cudaStream_t stream) {
  if (!a_mn && !b_mn) return launch_gemm<BN, false, false>(tA, tB, tA2, tB2, p, sm_count, stream);
  if (!a_mn && b_mn) return launch_gemm<BN, false, true>(tA, tB, tA2, tB2, p, sm_count, stream);
  if (a_mn && !b_mn) return launch_gemm<BN, true, false>(tA, tB, tA2, tB2, p, sm_count, stream);
  return launch_gemm<BN, true, true>(tA, tB, tA2, tB2, p, sm_count, stream);
}

int g_sm_count = 0;

struct PrefetchArgs {
  const unsigned long long* peer_bases = nullptr;  // device array
  unsigned long long shard_offset = 0, shard_bytes = 0;
  void* dst = nullptr;
  int world = 0;
  int ctas = 0;
};

int sm_count() {
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (g_sm_count <= 0) g_sm_count = 148;
  }
  return g_sm_count;
}

int fill_prefetch(GemmParams& p, const PrefetchArgs* pf) {
  p.g_ctas = 0;
  if (pf == nullptr || pf->ctas <= 0) return 0;
  if (pf->world < 1 || pf->shard_bytes == 0 || pf->shard_bytes % GATHER_CHUNK) return -7;
  p.g_ctas = pf->ctas;
  p.g_world = pf->world;
  p.g_peer_bases = pf->peer_bases;
  p.g_shard_offset = pf->shard_offset;
  p.g_shard_bytes = pf->shard_bytes;
  p.g_total_bytes = pf->shard_bytes * (unsigned long long)pf->world;
  p.g_dst = reinterpret_cast<unsigned char*>(pf->dst);
  return 0;
}

int gemm_entry(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn,
               void* C, long long ldc, const void* Cin, long long ldcin, int M, int N, int K,
               const void* A2, long long lda2, const void* B2, long long ldb2, int K2, float alpha,
               float beta, int out_mode, int splits, int bn, int* status, void* stream,
               const PrefetchArgs* pf) {
  if (M <= 0 || N <= 0 || (K <= 0 && K2 <= 0)) return 0;
  if ((lda & 7) || (ldb & 7) || (K2 > 0 && ((lda2 & 7) || (ldb2 & 7)))) return -2;
  if (splits < 1) splits = 1;
  if (splits > 1 && out_mode != 2) return -3;
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
  p.group_m = 8;
  if ((rc = fill_prefetch(p, pf)) != 0) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (bn) {
    case 64:
      return dispatch_major<64>(a_mn, b_mn, tA, tB, tA2, tB2, p, sm_count(), st);
    case 128:
      return dispatch_major<128>(a_mn, b_mn, tA, tB, tA2, tB2, p, sm_count(), st);
    case 256:
      return dispatch_major<256>(a_mn, b_mn, tA, tB, tA2, tB2, p, sm_count(), st);
    default:
      return -5;
  }
}

// stand-alone all-gather: every CTA is a gather CTA (used when nothing was prefetched)
__global__ void __launch_bounds__(kThreads, 1) gather_only_kernel(const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + GATHER_WARPS * GATHER_SLOTS * GATHER_CHUNK);
  gather_cta_body(p, blockIdx.x, gridDim.x, smem, bars);
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

// Same GEMM, plus `pf_ctas` trailing CTAs that all-gather a row-sharded matrix into `pf_dst`
// while the GEMM runs: rank r's shard (pf_shard_bytes bytes) lives at
// pf_peer_bases[r] + pf_shard_offset; pf_peer_bases is a DEVICE array of `pf_world` peer-mapped
// arena addresses. The gathered matrix is complete when the kernel has finished.
extern "C" int axb_gemm_bf16_prefetch(const void* A, long long lda, int a_mn, const void* B,
                                      long long ldb, int b_mn, void* C, long long ldc,
                                      const void* Cin, long long ldcin, int M, int N, int K,
                                      const void* A2, long long lda2, const void* B2,
                                      long long ldb2, int K2, float alpha, float beta,
                                      int out_mode, int splits, int bn,
                                      const unsigned long long* pf_peer_bases,
                                      unsigned long long pf_shard_offset,
                                      unsigned long long pf_shard_bytes, int pf_world, void* pf_dst,
                                      int pf_ctas, int* status, void* stream) {
  PrefetchArgs pf;
  pf.peer_bases = pf_peer_bases;
  pf.shard_offset = pf_shard_offset;
  pf.shard_bytes = pf_shard_bytes;
  pf.world = pf_world;
  pf.dst = pf_dst;
  pf.ctas = pf_ctas;
  return gemm_entry(A, lda, a_mn, B, ldb, b_mn, C, ldc, Cin, ldcin, M, N, K, A2, lda2, B2, ldb2, K2,
                    alpha, beta, out_mode, splits, bn, status, stream, &pf);
}

// GEMM whose epilogue all-reduces the result over NVLink: every rank adds its partial product
// into the symmetric bf16 buffer of every rank (pre-zeroed; `red_mc` = multicast address of that
// buffer, or NULL to use plain peer atomics through the HOST array red_ptrs[red_world]). The sum
// is complete on a rank once all ranks have finished the kernel (barrier afterwards).
extern "C" int axb_gemm_bf16_allreduce(const void* A, long long lda, int a_mn, const void* B, long long ldb,
                                       int b_mn, long long ldc, int M, int N, int K, const void* A2,
                                       long long lda2, const void* B2, long long ldb2, int K2, float alpha,
                                       int bn, void* red_mc, const unsigned long long* red_ptrs, int red_world,
                                       int* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N & 7) || (ldc & 7) || red_world < 1 || red_world > 8) return -2;
  if ((lda & 7) || (ldb & 7) || (K2 > 0 && ((lda2 & 7) || (ldb2 & 7)))) return -2;
  CUtensorMap tA, tB, tA2, tB2;
  int rc = 0;
  rc |= a_mn ? axb_make_tmap_2d(&tA, A, K, M, lda, 64, 64) : axb_make_tmap_2d(&tA, A, M, K, lda, BM, 64);
  rc |= b_mn ? axb_make_tmap_2d(&tB, B, K, N, ldb, 64, 64) : axb_make_tmap_2d(&tB, B, N, K, ldb, bn, 64);
  if (K2 > 0) {
    rc |= a_mn ? axb_make_tmap_2d(&tA2, A2, K2, M, lda2, 64, 64) : axb_make_tmap_2d(&tA2, A2, M, K2, lda2, BM, 64);
    rc |= b_mn ? axb_make_tmap_2d(&tB2, B2, K2, N, ldb2, 64, 64) : axb_make_tmap_2d(&tB2, B2, N, K2, ldb2, bn, 64);
  } else {
    tA2 = tA;
    tB2 = tB;
  }
  if (rc) return -4;
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K; p.K2 = K2 > 0 ? K2 : 0;
  p.ldc = ldc; p.alpha = alpha; p.splits = 1; p.status = status; p.group_m = 8;
  p.out_mode = red_mc ? 3 : 4;
  p.red_mc = red_mc;
  p.red_world = red_world;
  for (int i = 0; i < red_world; ++i) p.red_ptrs[i] = red_ptrs[i];
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (bn) {
    case 64: return dispatch_major<64>(a_mn, b_mn, tA, tB, tA2, tB2, p, sm_count(), st);
    case 128: return dispatch_major<128>(a_mn, b_mn, tA, tB, tA2, tB2, p, sm_count(), st);
    case 256: return dispatch_major<256>(a_mn, b_mn, tA, tB, tA2, tB2, p, sm_count(), st);
    default: return -5;
  }
}

// GEMM + two-shot all-reduce in one launch. Every rank stores its partial product (bf16) into its
// own symmetric buffer `C` (ldc = N) and `r_ctas` reducer CTAs sum each 128-row block over the
// ranks as soon as it is complete everywhere, writing the sum into every rank's buffer.
// red_mc: multicast address of the buffer (NULL = plain peer loads / stores through red_ptrs);
// cnt_ptrs: HOST array of the ranks' int32 [ceil(M / 128)] completion counters (zero before the
// first use; the kernel re-arms them). The sum is complete on a rank once all ranks have finished
// the kernel (barrier afterwards).
extern "C" int axb_gemm_bf16_allreduce2(const void* A, long long lda, int a_mn, const void* B, long long ldb,
                                        int b_mn, void* C, long long ldc, int M, int N, int K, const void* A2,
                                        long long lda2, const void* B2, long long ldb2, int K2, float alpha, int bn,
                                        void* red_mc, const unsigned long long* red_ptrs,
                                        const unsigned long long* cnt_ptrs, int red_rank, int red_world, int r_ctas,
                                        int* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N & 7) || (ldc & 7) || red_world < 1 || red_world > 8 || r_ctas < 1) return -2;
  if ((lda & 7) || (ldb & 7) || (K2 > 0 && ((lda2 & 7) || (ldb2 & 7)))) return -2;
  CUtensorMap tA, tB, tA2, tB2;
  int rc = 0;
  rc |= a_mn ? axb_make_tmap_2d(&tA, A, K, M, lda, 64, 64) : axb_make_tmap_2d(&tA, A, M, K, lda, BM, 64);
  rc |= b_mn ? axb_make_tmap_2d(&tB, B, K, N, ldb, 64, 64) : axb_make_tmap_2d(&tB, B, N, K, ldb, bn, 64);
  if (K2 > 0) {
    rc |= a_mn ? axb_make_tmap_2d(&tA2, A2, K2, M, lda2, 64, 64) : axb_make_tmap_2d(&tA2, A2, M, K2, lda2, BM, 64);
    rc |= b_mn ? axb_make_tmap_2d(&tB2, B2, K2, N, ldb2, 64, 64) : axb_make_tmap_2d(&tB2, B2, N, K2, ldb2, bn, 64);
  } else {
    tA2 = tA;
    tB2 = tB;
  }
  if (rc) return -4;
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K; p.K2 = K2 > 0 ? K2 : 0;
  p.C = C; p.ldc = ldc; p.alpha = alpha; p.splits = 1; p.status = status; p.group_m = 8;
  p.out_mode = 5;
  p.red_mc = red_mc;
  p.red_world = red_world;
  p.red_rank = red_rank;
  p.r_ctas = r_ctas;
  for (int i = 0; i < red_world; ++i) {
    p.red_ptrs[i] = red_ptrs[i];
    p.cnt_ptrs[i] = cnt_ptrs[i];
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (bn) {
    case 64: return dispatch_major<64>(a_mn, b_mn, tA, tB, tA2, tB2, p, sm_count(), st);
    case 128: return dispatch_major<128>(a_mn, b_mn, tA, tB, tA2, tB2, p, sm_count(), st);
    case 256: return dispatch_major<256>(a_mn, b_mn, tA, tB, tA2, tB2, p, sm_count(), st);
    default: return -5;
  }
}

// Stand-alone all-gather of a row-sharded matrix into `dst` with `ctas` CTAs (0 = one per SM).
extern "C" int axb_allgather_rows(const unsigned long long* peer_bases,
                                  unsigned long long shard_offset, unsigned long long shard_bytes,
                                  int world, void* dst, int ctas, int* status, void* stream) {
  PrefetchArgs pf;
  pf.peer_bases = peer_bases;
  pf.shard_offset = shard_offset;
  pf.shard_bytes = shard_bytes;
  pf.world = world;
  pf.dst = dst;
  pf.ctas = ctas > 0 ? ctas : sm_count();
  GemmParams p = {};
  p.status = status;
  int rc = fill_prefetch(p, &pf);
  if (rc) return rc;
  constexpr int smem_bytes = GATHER_WARPS * GATHER_SLOTS * GATHER_CHUNK + 1024 + 256;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gather_only_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  gather_only_kernel<<<pf.ctas, kThreads, smem_bytes, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  return (int)cudaGetLastError();
}

// =================================================================================================
// CTA-pair variant: 256 x 256 output tile per cluster of two CTAs (tcgen05.mma.cta_group::2).
// Each CTA stages its own 128 rows of A and its own 128 rows (columns of C) of B, so a k block
// costs 32 KB of shared memory per CTA instead of 48 KB: six pipeline stages instead of four and
// half the B traffic per FLOP. Rank 0 of the pair issues every MMA; both CTAs run a TMA producer
// and four epilogue warps on their own half of the accumulator.
// =================================================================================================
namespace {

constexpr int P_STAGES = 6;
constexpr int P_A_BYTES = 128 * BK * 2;       // 16 KB
constexpr int P_B_BYTES = 128 * BK * 2;       // 16 KB (this CTA's half of the 256-wide B tile)
constexpr int P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;
constexpr int P_EPI_BYTES = 4 * 2 * 4096;     // per epilogue warp: two staging slots of 32 rows x 128 bytes
constexpr int P_SMEM_BYTES = P_STAGES * P_STAGE_BYTES + P_EPI_BYTES + 1024 + 256;
constexpr int P_TMEM_COLS = 512;              // 2 accumulator stages x 256 columns

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                          const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2,
                          const __grid_constant__ CUtensorMap tmE0, const __grid_constant__ CUtensorMap tmE1,
                          const __grid_constant__ CUtensorMap tmE2, const __grid_constant__ CUtensorMap tmE3,
                          const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + P_STAGES * P_A_BYTES;
  uint8_t* sEpi = smem + P_STAGES * P_STAGE_BYTES;   // 1024-byte aligned (stages are 32 KB each)
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + P_STAGES * P_STAGE_BYTES + P_EPI_BYTES);
  uint64_t* full_bar = bars;                       // used in rank 0 only: both CTAs' loads of the stage
  uint64_t* empty_bar = bars + P_STAGES;           // one per CTA, signalled by the pair commit
  uint64_t* tfull_bar = bars + 2 * P_STAGES;       // one per CTA
  uint64_t* tempty_bar = bars + 2 * P_STAGES + 2;  // used in rank 0 only (8 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * P_STAGES + 4);
  uint64_t* epi_bar = bars + 24;                   // [epilogue warp][slot]: "gate|up chunk landed" (GLU backward)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_workers = (int)gridDim.x - p.g_ctas;  // even; gather CTAs come in whole clusters
  if ((int)blockIdx.x >= n_workers) {
    gather_cta_body(p, (int)blockIdx.x - n_workers, p.g_ctas, smem, bars);
    return;
  }
  const uint32_t rank = cluster_ctarank();
  const int cluster_id = blockIdx.x >> 1;
  const int n_clusters = n_workers >> 1;

  const int num_m = (p.M + 255) / 256;
  const int num_n = p.epi == 1 ? (p.N + 127) / 128 : (p.N + 255) / 256;
  const int nk_main = (p.K + BK - 1) / BK;
  const int nk_ext = (p.K2 + BK - 1) / BK;
  const int nk_total = nk_main + nk_ext;
  const int total_tiles = num_m * num_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tfull_bar[s], 1);
      mbar_init(&tempty_bar[s], 8);
    }
    for (int s = 0; s < 8; ++s) mbar_init(&epi_bar[s], 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 2) {
    tmem_alloc_pair(tmem_slot, P_TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();  // barriers of both CTAs are initialised before any remote arrive / TMA credit
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < total_tiles && ok; tile += n_clusters) {
        int m_blk, n_blk, split;
        decode_tile(tile, num_m, num_n, 1, m_blk, n_blk, split, p.group_m);
        for (int kb = 0; kb < nk_total; ++kb) {
          if (!mbar_wait_backoff(&empty_bar[stage], phase ^ 1, p.status, AXB_TIMEOUT_EMPTY, p.prod_sleep_ns)) {
            ok = false;
            break;
          }
          // One "full" barrier per stage, in the leader CTA: the leader expects the bytes of BOTH CTAs'
          // loads, and the partner's loads credit that barrier directly (cta_group::2 TMA). No relay,
          // no remote arrive, no fence on the critical path.
          const uint32_t fb = mapa_u32(smem_u32(&full_bar[stage]), 0);
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * P_STAGE_BYTES);
          const bool ext = kb >= nk_main;
          const CUtensorMap* ma = ext ? &tmA2 : &tmA;
          const CUtensorMap* mb = ext ? &tmB2 : &tmB;
          const int k0 = (ext ? kb - nk_main : kb) * BK;
          uint8_t* a_dst = sA + stage * P_A_BYTES;
          uint8_t* b_dst = sB + stage * P_B_BYTES;
          const int m0 = m_blk * 256 + (int)rank * 128;
          const int n0 = p.epi == 1 ? (int)rank * p.N + n_blk * 128 : n_blk * 256 + (int)rank * 128;
          if (!A_MN) {
            tma_load_2d_pair(a_dst, ma, fb, k0, m0);
          } else {
            tma_load_2d_pair(a_dst, ma, fb, m0, k0);
            tma_load_2d_pair(a_dst + 8192, ma, fb, m0 + 64, k0);
          }
          if (!B_MN) {
            tma_load_2d_pair(b_dst, mb, fb, k0, n0);
          } else {
            tma_load_2d_pair(b_dst, mb, fb, n0, k0);
            tma_load_2d_pair(b_dst + 8192, mb, fb, n0 + 64, k0);
          }
          if (++stage == P_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (rank 0 only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(256, 256, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < total_tiles && ok; tile += n_clusters, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait_spin(&tempty_bar[acc], acc_phase ^ 1, p.status, AXB_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * 256;
        for (int kb = 0; kb < nk_total; ++kb) {
          if (!mbar_wait_spin(&full_bar[stage], phase, p.status, AXB_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * P_A_BYTES);
          const uint32_t b_addr = smem_u32(sB + stage * P_B_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            const uint64_t da = A_MN ? make_smem_desc_sw128(a_addr + kk * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(a_addr + kk * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(b_addr + kk * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(b_addr + kk * 32, 16, 1024);
            umma_f16_pair(d_tmem, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit_pair_mc(&empty_bar[stage]);  // frees the stage in both CTAs (commit multicast)
          if (++stage == P_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit_pair_mc(&tfull_bar[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (both CTAs)
    const int lane_group = warp & 3;
    uint8_t* my_epi = sEpi + lane_group * 8192;   // this warp's two staging slots
    int slot = 0;
    int q = 0;                                    // GLU backward: running chunk counter (slot and barrier phase)
    int it = 0;
    bool ok = true;
    for (int tile = cluster_id; tile < total_tiles && ok; tile += n_clusters, ++it) {
      int m_blk, n_blk, split;
      decode_tile(tile, num_m, num_n, 1, m_blk, n_blk, split, p.group_m);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (p.epi == 2 && lane == 0) {
        // first gate|up chunk of this tile: requested now, it lands while the MMAs of the tile still run
        bulk_wait_group_read<0>();
        uint8_t* dst = my_epi + (q & 1) * 4096;
        uint64_t* eb = &epi_bar[lane_group * 2 + (q & 1)];
        const int r0 = m_blk * 256 + (int)rank * 128 + lane_group * 32;
        mbar_expect_tx(eb, 4096);
        tma_load_2d(dst, &tmE2, eb, n_blk * 256, r0);
        tma_load_2d(dst + 2048, &tmE3, eb, n_blk * 256, r0);
      }
      if (!mbar_wait_backoff(&tfull_bar[acc], acc_phase, p.status, AXB_TIMEOUT_TMEM_FULL, p.epi_sleep_ns)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const long long row = (long long)m_blk * 256 + rank * 128 + lane_group * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t t_addr = tmem_base + (uint32_t(lane_group * 32) << 16) + acc * 256;
      const int warp_row0 = m_blk * 256 + (int)rank * 128 + lane_group * 32;   // first row of this warp's 32
      const bool warp_rows = warp_row0 < p.M;
      // stage one 32 x 64 bf16 tile (this warp's rows) and hand it to the TMA store engine
      auto put128 = [&](const CUtensorMap* map, const uint4 (&w)[8], int col0) {
        uint8_t* tile = my_epi + slot * 4096;
        if (lane == 0) bulk_wait_group_read<1>();   // the store that last read this slot is done with it
        __syncwarp();
        stage_row128(tile, lane, w);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(map, tile, col0, warp_row0);
          bulk_commit_group();
        }
        slot ^= 1;
      };
      if (p.epi == 1) {
        // GLU forward: columns [0, 128) of the accumulator are gate, [128, 256) the matching up columns
        const int I = p.N;
        const bool lim = p.glu_limit > 0.f;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t r0[32], r1[32];
          uint4 gw[8], uw[8];
          tmem_ld_32x32(t_addr + c * 64, r0);
          tmem_ld_32x32(t_addr + c * 64 + 32, r1);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            gw[j] = pack8(r0 + 8 * j, p.alpha);
            gw[4 + j] = pack8(r1 + 8 * j, p.alpha);
          }
          tmem_ld_32x32(t_addr + 128 + c * 64, r0);
          tmem_ld_32x32(t_addr + 128 + c * 64 + 32, r1);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uw[j] = pack8(r0 + 8 * j, p.alpha);
            uw[4 + j] = pack8(r1 + 8 * j, p.alpha);
          }
          const int col0 = n_blk * 128 + c * 64;
          if (!warp_rows || col0 >= I) continue;
          if (p.C) {
            put128(&tmE0, gw, col0);
            put128(&tmE1, uw, col0);
          }
          // h from the bf16-rounded gate / up, so that the backward pass sees the same values
          uint4 hw[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t g4[4] = {gw[j].x, gw[j].y, gw[j].z, gw[j].w};
            const uint32_t u4[4] = {uw[j].x, uw[j].y, uw[j].z, uw[j].w};
            uint32_t h4[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 g = unpack_bf16x2(g4[e]), u = unpack_bf16x2(u4[e]);
              const float ga = lim ? fminf(g.x, p.glu_limit) : g.x, gb = lim ? fminf(g.y, p.glu_limit) : g.y;
              const float ua = lim ? fminf(fmaxf(u.x, -p.glu_limit), p.glu_limit) : u.x;
              const float ub = lim ? fminf(fmaxf(u.y, -p.glu_limit), p.glu_limit) : u.y;
              h4[e] = pack_bf16x2(glu_act(ga, p.glu_kind) * ua, glu_act(gb, p.glu_kind) * ub);
            }
            hw[j] = make_uint4(h4[0], h4[1], h4[2], h4[3]);
          }
          put128(&tmE2, hw, col0);
        }
      } else if (p.epi == 2) {
        // GLU backward: the accumulator is dh. gate | up chunks (32 rows x 32 columns each) arrive by
        // TMA in one of two staging slots, one chunk ahead of the arithmetic; d_gate | d_up overwrite
        // them in place and leave by TMA stores.
        const int I = p.N;
        const bool lim = p.glu_limit > 0.f;
        const float L = p.glu_limit;
#pragma unroll 1
        for (int c = 0; c < 8; ++c, ++q) {
          const int col0 = n_blk * 256 + c * 32;
          const int s_cur = q & 1;
          uint8_t* tile = my_epi + s_cur * 4096;
          if (c < 7 && lane == 0) {
            // the other slot was last read by the stores of chunk q-1
            bulk_wait_group_read<0>();
            uint8_t* nxt = my_epi + (s_cur ^ 1) * 4096;
            uint64_t* nb = &epi_bar[lane_group * 2 + (s_cur ^ 1)];
            mbar_expect_tx(nb, 4096);
            tma_load_2d(nxt, &tmE2, nb, col0 + 32, warp_row0);
            tma_load_2d(nxt + 2048, &tmE3, nb, col0 + 32, warp_row0);
          }
          uint32_t r[32];
          tmem_ld_32x32(t_addr + c * 32, r);
          tmem_ld_wait();
          if (!mbar_wait(&epi_bar[lane_group * 2 + s_cur], (uint32_t)((q >> 1) & 1), p.status, AXB_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          const int sw = (lane >> 1) & 3;
          uint8_t* grow = tile + lane * 64;
          uint8_t* urow = tile + 2048 + lane * 64;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4* gp = reinterpret_cast<uint4*>(grow + ((j ^ sw) << 4));
            uint4* up = reinterpret_cast<uint4*>(urow + ((j ^ sw) << 4));
            const uint4 gq = *gp, uq = *up;
            const uint32_t g4[4] = {gq.x, gq.y, gq.z, gq.w};
            const uint32_t u4[4] = {uq.x, uq.y, uq.z, uq.w};
            uint32_t og[4], ou[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 g = unpack_bf16x2(g4[e]), u = unpack_bf16x2(u4[e]);
              const float gv[2] = {g.x, g.y}, uv[2] = {u.x, u.y};
              float a[2], b[2];
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const float d = __uint_as_float(r[8 * j + 2 * e + h]) * p.alpha;
                const bool g_in = !lim || gv[h] <= L;
                const bool u_in = !lim || (uv[h] >= -L && uv[h] <= L);
                const float gc = g_in ? gv[h] : L;
                const float uc = u_in ? uv[h] : (uv[h] > 0.f ? L : -L);
                float dact;
                const float act = glu_act_and_grad(gc, p.glu_kind, dact);
                a[h] = g_in ? d * uc * dact : 0.f;
                b[h] = u_in ? d * act : 0.f;
              }
              og[e] = pack_bf16x2(a[0], a[1]);
              ou[e] = pack_bf16x2(b[0], b[1]);
            }
            *gp = make_uint4(og[0], og[1], og[2], og[3]);
            *up = make_uint4(ou[0], ou[1], ou[2], ou[3]);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (warp_rows && col0 < I) {
              tma_store_2d(&tmE0, tile, col0, warp_row0);
              tma_store_2d(&tmE1, tile + 2048, col0, warp_row0);
            }
            bulk_commit_group();
          }
        }
        if (!ok) break;
      } else if (p.tma_store) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(t_addr + c * 64, r0);
          tmem_ld_32x32(t_addr + c * 64 + 32, r1);
          tmem_ld_wait();
          const int col0 = n_blk * 256 + c * 64;
          if (!warp_rows || col0 >= p.N) continue;
          uint4 w[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            w[j] = pack8(r0 + 8 * j, p.alpha);
            w[4 + j] = pack8(r1 + 8 * j, p.alpha);
          }
          put128(&tmE0, w, col0);
        }
      } else
#pragma unroll 1
      for (int c = 0; c < 8; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_addr + c * 32, r);
        tmem_ld_wait();
        const int col0 = n_blk * 256 + c * 32;
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
        } else {
          float* crow = reinterpret_cast<float*>(p.C) + row * p.ldc + col0;
          const float* irow = p.Cin ? reinterpret_cast<const float*>(p.Cin) + row * p.ldcin + col0 : nullptr;
          if (full_chunk && (p.ldc & 3) == 0 && (!irow || (p.ldcin & 3) == 0)) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              float4 o = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
              if (irow) {
                const float4 in = *reinterpret_cast<const float4*>(irow + q * 4);
                o.x += p.beta * in.x;
                o.y += p.beta * in.y;
                o.z += p.beta * in.z;
                o.w += p.beta * in.w;
              }
              *reinterpret_cast<float4*>(crow + q * 4) = o;
            }
          } else {
            for (int j = 0; j < 32 && col0 + j < p.N; ++j) crow[j] = v[j] + (irow ? p.beta * irow[j] : 0.f);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tempty_bar[acc]), 0));
    }
    if (lane == 0) bulk_wait_group<0>();   // staged tiles are in global memory before shared memory goes away
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync();  // neither CTA may leave (and release smem / TMEM) while its partner still signals it
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, P_TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN>
int launch_pair(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tA2, const CUtensorMap& tB2,
                const CUtensorMap& tE0, const CUtensorMap& tE1, const CUtensorMap& tE2, const CUtensorMap& tE3,
                GemmParams p, int sms, cudaStream_t stream) {
  auto kern = gemm_bf16_pair_kernel<A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  p.g_ctas &= ~1;  // whole clusters only
  const int tiles = ((p.M + 255) / 256) * (p.epi == 1 ? (p.N + 127) / 128 : (p.N + 255) / 256);
  int workers = (sms - p.g_ctas) & ~1;
  if (2 * tiles < workers) workers = 2 * tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(workers + p.g_ctas, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = P_SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, kern, tA, tB, tA2, tB2, tE0, tE1, tE2, tE3, p);
}

}  // namespace

// CTA-pair GEMM (same contract as axb_gemm_bf16_prefetch with bn = 256, splits = 1, out_mode 0/1).
// epi = 0: plain. epi = 1 (GLU forward): B is the [2I, K] gate|up weight (B2 the matching [2I, K2]
// LoRA factor), N = I; C (optional) receives gate|up [M, 2I], H receives act(gate) * up [M, I].
// epi = 2 (GLU backward): N = I, the product is dh [M, I]; Cin holds gate|up [M, 2I] and C receives
// d_gate | d_up [M, 2I] (C may alias Cin). glu_kind 0 = SiLU, 1 = GELU(tanh); glu_limit > 0 clamps.
static int pair_entry(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn,
                      void* C, long long ldc, const void* Cin, long long ldcin, int M, int N, int K,
                      const void* A2, long long lda2, const void* B2, long long ldb2, int K2,
                      float alpha, float beta, int out_mode, int epi, int glu_kind, float glu_limit, void* H,
                      long long ldh, const unsigned long long* pf_peer_bases, unsigned long long pf_shard_offset,
                      unsigned long long pf_shard_bytes, int pf_world, void* pf_dst, int pf_ctas,
                      int* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (ldb & 7) || (K2 > 0 && ((lda2 & 7) || (ldb2 & 7)))) return -2;
  if (out_mode != 0 && out_mode != 1) return -3;
  if (epi < 0 || epi > 2) return -3;
  if (epi == 1 && (b_mn || out_mode != 0 || H == nullptr)) return -3;
  if (epi == 2 && (out_mode != 0 || Cin == nullptr || C == nullptr)) return -3;
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (epi != 0) {  // the GLU epilogues move whole 16-byte vectors and 32-column chunks
    if ((N & 31) || (ldc & 7) || !al16(C) || (epi == 1 && ((ldh & 7) || !al16(H))) ||
        (epi == 2 && ((ldcin & 7) || !al16(Cin))))
      return -2;
  }
  const int n_rows_b = epi == 1 ? 2 * N : N;   // rows of the stored B (K-major) / columns (MN-major)
  CUtensorMap tA, tB, tA2, tB2;
  int rc = 0;
  rc |= a_mn ? axb_make_tmap_2d(&tA, A, K, M, lda, 64, 64) : axb_make_tmap_2d(&tA, A, M, K, lda, 128, 64);
  rc |= b_mn ? axb_make_tmap_2d(&tB, B, K, n_rows_b, ldb, 64, 64) : axb_make_tmap_2d(&tB, B, n_rows_b, K, ldb, 128, 64);
  if (K2 > 0) {
    rc |= a_mn ? axb_make_tmap_2d(&tA2, A2, K2, M, lda2, 64, 64) : axb_make_tmap_2d(&tA2, A2, M, K2, lda2, 128, 64);
    rc |= b_mn ? axb_make_tmap_2d(&tB2, B2, K2, n_rows_b, ldb2, 64, 64)
               : axb_make_tmap_2d(&tB2, B2, n_rows_b, K2, ldb2, 128, 64);
  } else {
    tA2 = tA;
    tB2 = tB;
  }
  // epilogue maps: staging tiles of 32 rows x 64 columns (128-byte swizzle), or 32 x 32 (64-byte swizzle)
  // for the GLU backward pass
  CUtensorMap tE0 = tA, tE1 = tA, tE2 = tA, tE3 = tA;
  int tma_store = 0;
  const __nv_bfloat16* Cb = reinterpret_cast<const __nv_bfloat16*>(C);
  if (epi == 0) {
    if (g_pair_tma_store && out_mode == 0 && Cin == nullptr && (ldc & 7) == 0 && al16(C)) {
      rc |= axb_make_tmap_2d(&tE0, C, M, N, ldc, 32, 64);
      tma_store = 1;
    }
  } else if (epi == 1) {
    if (C) {
      rc |= axb_make_tmap_2d(&tE0, Cb, M, N, ldc, 32, 64);
      rc |= axb_make_tmap_2d(&tE1, Cb + N, M, N, ldc, 32, 64);
    }
    rc |= axb_make_tmap_2d(&tE2, H, M, N, ldh, 32, 64);
  } else {
    const __nv_bfloat16* Gb = reinterpret_cast<const __nv_bfloat16*>(Cin);
    rc |= axb_make_tmap_2d(&tE0, Cb, M, N, ldc, 32, 32, 2, false, true);
    rc |= axb_make_tmap_2d(&tE1, Cb + N, M, N, ldc, 32, 32, 2, false, true);
    rc |= axb_make_tmap_2d(&tE2, Gb, M, N, ldcin, 32, 32, 2, false, true);
    rc |= axb_make_tmap_2d(&tE3, Gb + N, M, N, ldcin, 32, 32, 2, false, true);
  }
  if (rc) return -4;
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K; p.K2 = K2 > 0 ? K2 : 0;
  p.C = C; p.Cin = Cin; p.ldc = ldc; p.ldcin = ldcin;
  p.alpha = alpha; p.beta = beta; p.out_mode = out_mode; p.splits = 1; p.status = status;
  p.epi = epi; p.glu_kind = glu_kind; p.glu_limit = glu_limit; p.H = H; p.ldh = ldh;
  p.epi_sleep_ns = g_epi_sleep_ns; p.prod_sleep_ns = g_prod_sleep_ns;
  p.tma_store = tma_store;
  // Rasterisation band: `group_m` rows of 256-row tiles sweep over N together, so their A rows are read
  // from DRAM once (they stay in L2) while B is streamed once per band. Taller bands mean fewer passes
  // over B; the band's A rows (group_m x 256 x K bf16) have to fit the L2 share given to them.
  if (g_pair_group_m > 0) {
    p.group_m = g_pair_group_m;
  } else {
    const long long per_tile_row = 256LL * (K + (K2 > 0 ? K2 : 0)) * 2;
    long long g = ((long long)g_pair_band_mb << 20) / per_tile_row;
    p.group_m = (int)(g < 2 ? 2 : (g > 16 ? 16 : g));
  }
  PrefetchArgs pf;
  pf.peer_bases = pf_peer_bases; pf.shard_offset = pf_shard_offset; pf.shard_bytes = pf_shard_bytes;
  pf.world = pf_world; pf.dst = pf_dst; pf.ctas = pf_ctas;
  if ((rc = fill_prefetch(p, &pf)) != 0) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (!a_mn && !b_mn) return launch_pair<false, false>(tA, tB, tA2, tB2, tE0, tE1, tE2, tE3, p, sm_count(), st);
  if (!a_mn && b_mn) return launch_pair<false, true>(tA, tB, tA2, tB2, tE0, tE1, tE2, tE3, p, sm_count(), st);
  if (a_mn && !b_mn) return launch_pair<true, false>(tA, tB, tA2, tB2, tE0, tE1, tE2, tE3, p, sm_count(), st);
  return launch_pair<true, true>(tA, tB, tA2, tB2, tE0, tE1, tE2, tE3, p, sm_count(), st);
}

extern "C" int axb_gemm_bf16_pair(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn,
                                  void* C, long long ldc, const void* Cin, long long ldcin, int M, int N, int K,
                                  const void* A2, long long lda2, const void* B2, long long ldb2, int K2,
                                  float alpha, float beta, int out_mode,
                                  const unsigned long long* pf_peer_bases, unsigned long long pf_shard_offset,
                                  unsigned long long pf_shard_bytes, int pf_world, void* pf_dst, int pf_ctas,
                                  int* status, void* stream) {
  return pair_entry(A, lda, a_mn, B, ldb, b_mn, C, ldc, Cin, ldcin, M, N, K, A2, lda2, B2, ldb2, K2, alpha, beta,
                    out_mode, 0, 0, 0.f, nullptr, 0, pf_peer_bases, pf_shard_offset, pf_shard_bytes, pf_world, pf_dst,
                    pf_ctas, status, stream);
}

// CTA-pair GEMM with a GLU epilogue (see pair_entry): the SwiGLU / GeGLU of an MLP folded into the
// gate|up projection (forward) and into the input-gradient GEMM of the down projection (backward),
// which the reference runs as separate Triton kernels (src/axolotl/kernels/swiglu.py:16-101,
// src/axolotl/kernels/geglu.py) between cuBLAS calls.
extern "C" int axb_gemm_bf16_pair_glu(const void* A, long long lda, int a_mn, const void* B, long long ldb, int b_mn,
                                      void* C, long long ldc, const void* Cin, long long ldcin, int M, int N, int K,
                                      const void* A2, long long lda2, const void* B2, long long ldb2, int K2,
                                      float alpha, int epi, int glu_kind, float glu_limit, void* H, long long ldh,
                                      const unsigned long long* pf_peer_bases, unsigned long long pf_shard_offset,
                                      unsigned long long pf_shard_bytes, int pf_world, void* pf_dst, int pf_ctas,
                                      int* status, void* stream) {
  if (epi != 1 && epi != 2) return -3;
  return pair_entry(A, lda, a_mn, B, ldb, b_mn, C, ldc, Cin, ldcin, M, N, K, A2, lda2, B2, ldb2, K2, alpha, 0.f, 0,
                    epi, glu_kind, glu_limit, H, ldh, pf_peer_bases, pf_shard_offset, pf_shard_bytes, pf_world, pf_dst,
                    pf_ctas, status, stream);
}

// Wait back-off of the CTA-pair kernel in nanoseconds (0 = busy spin): epilogue warps waiting for an
// accumulator, TMA producer waiting for a free stage.
extern "C" void axb_gemm_set_backoff(int epi_sleep_ns, int prod_sleep_ns) {
  g_epi_sleep_ns = epi_sleep_ns;
  g_prod_sleep_ns = prod_sleep_ns;
}

// Tuning of the CTA-pair kernel: 256-row tile rows per rasterisation band (0 = as many as fit band_mb
// MiB of A rows, between 2 and 16) and whether bf16 results leave through TMA tile stores (1) or
// per-thread row stores (0).
extern "C" void axb_gemm_set_pair_tuning(int group_m, int tma_store, int band_mb) {
  g_pair_group_m = group_m;          // 0: derive the band height from band_mb (MiB of A rows per band)
  g_pair_tma_store = tma_store;
  if (band_mb > 0) g_pair_band_mb = band_mb;
}
