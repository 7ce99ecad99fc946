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
// Per k block the TMA producer brings the bf16 A tiles and the PACKED weight tile (4 KB instead of 16 KB)
// into shared memory; four converter warps expand the nibbles and write the bf16 tile in the
// 128-byte-swizzled layout tcgen05.mma reads; the MMA warp accumulates in TMEM; four epilogue warps store
// the result. One decoded weight tile feeds TWO 128-row blocks of the same expert (256 rows per pass), which
// halves the decode work per FLOP. The decode builds, per 16-value scale group, the eight products
// |e2m1| x scale as bf16 (one fp32 multiply for 1.5 x scale; the power-of-two multiples are exponent
// offsets of the same two roundings) and picks them with byte permutes, about 2.6 instructions per value.
// The decoded values are bit-identical to nvfp4_dequant_kernel's, so the product equals
// dequantise-then-GEMM exactly, at a quarter of the weight traffic and without the bf16 scratch. This is the role the Marlin W4A16 grouped kernel and the
// dequantise-into-a-chunk path play in the reference
// (src/axolotl/integrations/kernels/libs/scattermoe_lora/marlin_w4a16/_csrc/libtorch_stable/moe/marlin_moe_wna16/marlin_template.h:251,
//  src/axolotl/integrations/kernels/libs/scattermoe_lora/grouped_train.py:446-596).
#include "axb_common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int BK = 64;
constexpr int W4_CONV_WARPS = 8;
constexpr int W4_THREADS = 192 + 32 * W4_CONV_WARPS;   // TMA, MMA, 4 epilogue warps, 8 converter warps
constexpr int W4_STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;   // one 128-row A tile; a stage holds two
constexpr int B_BYTES = BN * BK * 2;
constexpr int RAW_BYTES = 4096;   // FWD: 128 rows x 32 bytes; DX: 64 rows x 64 bytes
constexpr int W4_SMEM = W4_STAGES * (2 * A_BYTES + B_BYTES + RAW_BYTES) + 1024 + 256;

// E4M3 byte -> fp32, branch free: the 7 magnitude bits placed at the top of an fp32 mantissa / the bottom of
// its exponent give value x 2^-120 (subnormal inputs included), and 0x7F / 0xFF are NaN. Same value as
// the table-free decode of nvfp4_dequant_kernel.
AXB_DEVICE float e4m3_to_float(uint32_t v) {
  const uint32_t mag = v & 0x7Fu;
  float f = __uint_as_float(mag << 20) * 1.329227995784916e36f;   // 2^120
  f = mag == 0x7Fu ? __int_as_float(0x7fc00000) : f;
  return __uint_as_float(__float_as_uint(f) | ((v & 0x80u) << 24));
}
AXB_DEVICE uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
// The eight bf16 products |code| x s of one scale group, split into low-byte and high-byte tables for prmt.
// |code| = 0, .5, 1, 1.5, 2, 3, 4, 6: bf16(fp32(m x s)) for m a power of two is bf16(s) with the exponent
// moved, and 3 s, 6 s are 1.5 s with the exponent moved, so two roundings give all eight (same bits as
// rounding each fp32 product) as long as no exponent leaves the normal range; otherwise multiply them out.
struct Lut {
  uint32_t L0, L1, H0, H1;
};
AXB_DEVICE Lut make_lut(float s) {
  const uint32_t P23 = pack_bf16x2(s, 1.5f * s);   // low half: 1 x s, high half: 1.5 x s
  uint32_t P01, P45, P67;
  if (((P23 >> 7) & 0x1FFu) - 2u < 0xFAu) {        // s positive, exponent in [2, 251]
    P01 = (P23 << 16) - 0x00800000u;               // (0, 0.5 s)
    P45 = P23 + 0x00800080u;                       // (2 s, 3 s)
    P67 = P23 + 0x01000100u;                       // (4 s, 6 s)
  } else {
    P01 = pack_bf16x2(0.f * s, 0.5f * s);
    P45 = pack_bf16x2(2.f * s, 3.f * s);
    P67 = pack_bf16x2(4.f * s, 6.f * s);
  }
  Lut t;
  t.L0 = prmt(P01, P23, 0x6420);
  t.H0 = prmt(P01, P23, 0x7531);
  t.L1 = prmt(P45, P67, 0x6420);
  t.H1 = prmt(P45, P67, 0x7531);
  return t;
}
// 8 packed codes (one 32-bit word, low nibble first) -> 8 bf16 in a 16-byte chunk
AXB_DEVICE uint4 decode8(uint32_t w, const Lut& t) {
  const uint32_t sel = w & 0x77777777u, selh = sel >> 16;
  const uint32_t sg = w & 0x88888888u, sg4 = sg << 4;   // sign of odd codes / even codes at bit 7 of byte i/2
  uint32_t lo = prmt(t.L0, t.L1, sel), hi = prmt(t.H0, t.H1, sel);
  hi ^= prmt(sg4, sg, 0x5140) & 0x80808080u;
  uint4 o;
  o.x = prmt(lo, hi, 0x5140);
  o.y = prmt(lo, hi, 0x7362);
  lo = prmt(t.L0, t.L1, selh);
  hi = prmt(t.H0, t.H1, selh);
  hi ^= prmt(sg4, sg, 0x7362) & 0x80808080u;
  o.z = prmt(lo, hi, 0x5140);
  o.w = prmt(lo, hi, 0x7362);
  return o;
}

struct W4Params {
  int N, K, K2;   // FWD: N output columns, K contraction. DX: N = output columns (the weight's K), K = contraction (the weight's N)
  int Wn, Wk;     // logical weight shape [Wn, Wk] per expert
  int E;
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

// One pass = one decoded weight tile stream against one or two 128-row blocks of the same expert.
struct Pass {
  int blk, two, e, n0;
};
// Tiles are (pair of consecutive row blocks, n block). Sub-pass 0 takes block 2p (and 2p+1 when it belongs to
// the same expert); sub-pass 1 exists only when block 2p+1 belongs to another expert.
AXB_DEVICE bool get_pass(const int* blk_expert, int n_blocks, int num_n, int E, int tile, int sub, Pass& ps) {
  const int pair = tile / num_n;
  const int b0 = 2 * pair, b1 = b0 + 1;
  int e0 = blk_expert[b0];
  const bool has1 = b1 < n_blocks;
  int e1 = has1 ? blk_expert[b1] : -1;
  if (!AXB_INDEX_OK(AXB_SITE_W4A16_EXPERT, e0, E)) e0 = 0;              // checked build: recorded, then a valid expert
  if (has1 && !AXB_INDEX_OK(AXB_SITE_W4A16_EXPERT, e1, E)) e1 = 0;
  ps.n0 = (tile - pair * num_n) * BN;
  if (sub == 0) {
    ps.blk = b0;
    ps.two = has1 && e1 == e0;
    ps.e = e0;
    return true;
  }
  if (!has1 || e1 == e0) return false;
  ps.blk = b1;
  ps.two = 0;
  ps.e = e1;
  return true;
}

template <bool DX>
__global__ void __launch_bounds__(W4_THREADS, 1)
    grouped_w4a16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmQ,
                         const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2,
                         const W4Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;                                   // [stage][2][128 x 64]
  uint8_t* sB = smem + W4_STAGES * 2 * A_BYTES;
  uint8_t* sRaw = sB + W4_STAGES * B_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sRaw + W4_STAGES * RAW_BYTES);
  uint64_t* raw_full = bars;                    // TMA landed: A tiles + packed weights (or the bf16 LoRA tile)
  uint64_t* full_bar = bars + W4_STAGES;        // converters done: the bf16 B tile is in place (one arrival per warp)
  uint64_t* empty_bar = bars + 2 * W4_STAGES;   // MMAs retired
  uint64_t* tfull_bar = bars + 3 * W4_STAGES;
  uint64_t* tempty_bar = bars + 3 * W4_STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * W4_STAGES + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_blocks = *p.n_blocks;
  const int num_n = (p.N + BN - 1) / BN;
  const int nk_main = (p.K + BK - 1) / BK, nk_ext = (p.K2 + BK - 1) / BK;
  const int nk = nk_main + nk_ext;
  const int total = ((n_blocks + 1) / 2) * num_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < W4_STAGES; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&full_bar[s], W4_CONV_WARPS);
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
    tmem_alloc(tmem_slot, 512);   // two accumulator slots of 2 x 128 columns
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
        for (int sub = 0; sub < 2 && ok; ++sub) {
          Pass ps;
          if (!get_pass(p.blk_expert, n_blocks, num_n, p.E, tile, sub, ps)) continue;
          const uint32_t a_bytes = ps.two ? 2 * A_BYTES : A_BYTES;
          for (int kb = 0; kb < nk; ++kb) {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, AXB_TIMEOUT_EMPTY)) {
              ok = false;
              break;
            }
            const bool ext = kb >= nk_main;
            uint8_t* a_dst = sA + stage * 2 * A_BYTES;
            const CUtensorMap* ma = ext ? &tmA2 : &tmA;
            const int ka = ext ? (kb - nk_main) * BK : kb * BK;
            mbar_expect_tx(&raw_full[stage], a_bytes + (ext ? B_BYTES : RAW_BYTES));
            tma_load_2d(a_dst, ma, &raw_full[stage], ka, ps.blk * BM);
            if (ps.two) tma_load_2d(a_dst + A_BYTES, ma, &raw_full[stage], ka, (ps.blk + 1) * BM);
            if (!ext) {
              if (!DX) tma_load_3d(sRaw + stage * RAW_BYTES, &tmQ, &raw_full[stage], kb * (BK / 2), ps.n0, ps.e);   // [128 n, 32 B of k]
              else tma_load_3d(sRaw + stage * RAW_BYTES, &tmQ, &raw_full[stage], ps.n0 / 2, kb * BK, ps.e);         // [64 n, 64 B of k]
            } else {
              uint8_t* b_dst = sB + stage * B_BYTES;
              if (!DX) {
                tma_load_3d(b_dst, &tmB2, &raw_full[stage], ka, ps.n0, ps.e);
              } else {
                tma_load_3d(b_dst, &tmB2, &raw_full[stage], ps.n0, ka, ps.e);
                tma_load_3d(b_dst + 8192, &tmB2, &raw_full[stage], ps.n0 + 64, ka, ps.e);
              }
            }
            if (++stage == W4_STAGES) {
              stage = 0;
              phase ^= 1;
            }
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
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        for (int sub = 0; sub < 2 && ok; ++sub) {
          Pass ps;
          if (!get_pass(p.blk_expert, n_blocks, num_n, p.E, tile, sub, ps)) continue;
          const int acc = it & 1;
          if (!mbar_wait(&tempty_bar[acc], ((it >> 1) & 1) ^ 1, p.status, AXB_TIMEOUT_TMEM_EMPTY)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * 2 * BN;
          for (int kb = 0; kb < nk; ++kb) {
            // raw_full: the TMA writes (A tiles, LoRA B tile) observed by this thread itself; full_bar: the decoded tile
            if (!mbar_wait(&raw_full[stage], phase, p.status, AXB_TIMEOUT_FULL) ||
                !mbar_wait(&full_bar[stage], phase, p.status, AXB_TIMEOUT_FULL)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t a_addr = smem_u32(sA + stage * 2 * A_BYTES), b_addr = smem_u32(sB + stage * B_BYTES);
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk) {
              const uint64_t db = DX ? make_smem_desc_sw128(b_addr + kk * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(b_addr + kk * 32, 16, 1024);
              const uint32_t accum = (kb > 0 || kk > 0) ? 1u : 0u;
              umma_f16(d_tmem, make_smem_desc_sw128(a_addr + kk * 32, 16, 1024), db, idesc, accum);
              if (ps.two) umma_f16(d_tmem + BN, make_smem_desc_sw128(a_addr + A_BYTES + kk * 32, 16, 1024), db, idesc, accum);
            }
            umma_commit(&empty_bar[stage]);
            if (++stage == W4_STAGES) {
              stage = 0;
              phase ^= 1;
            }
          }
          if (!ok) break;
          umma_commit(&tfull_bar[acc]);
          ++it;
        }
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------ converters: packed tile -> bf16 B tile
    // 256 threads; thread ct reads 16 packed bytes (32 codes, 2 scale groups) at raw + ct * 16 and writes four
    // 16-byte chunks of the swizzled bf16 tile. Two warps per scheduler hide each other's latencies.
    //   FWD: raw tile [128 n][32 B]: weight row n0 + ct / 2, codes 32 * (ct & 1) .. + 31 of k block kb
    //        -> K-major row ct / 2, chunks 4 * (ct & 1) .. + 3.
    //   DX : raw tile [64 wn][64 B]: weight row kb * 64 + ct / 4, columns n0 + 64 * half + 32 * part .. + 31
    //        (half = (ct >> 1) & 1, part = ct & 1) -> MN-major chunk block `half`, row ct / 4, chunks 4 * part .. + 3.
    // Shared-memory accesses are conflict free: the loads are contiguous, and the eight lanes of a store phase
    // hit eight different 16-byte chunk positions (rows differ in swizzle bits 0-1 or bit 0, `part` flips bit 2,
    // and in dX the odd half walks its chunks in the order 2, 3, 0, 1, which flips bit 1).
    const int ct = threadIdx.x - 192;   // 0..255
    const long long sc_row_bytes = p.Wk / 16;
    const int part = ct & 1;
    const int r = DX ? (ct >> 2) : (ct >> 1), half = DX ? ((ct >> 1) & 1) : 0;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
      for (int sub = 0; sub < 2 && ok; ++sub) {
        Pass ps;
        if (!get_pass(p.blk_expert, n_blocks, num_n, p.E, tile, sub, ps)) continue;
        const float g = p.pts[ps.e];
        const uint8_t* sc_base = p.scale + (long long)ps.e * p.Wn * sc_row_bytes;
        // Block scales (2 bytes per thread and k block) are fetched FOUR k blocks ahead: a global load that misses
        // the small L1 left beside 200 KB of shared memory takes longer than one k block. Forward: one 16-byte
        // load covers four k blocks of this thread's weight row; dX: a new weight row per k block.
        const bool vec_ok = !DX && (sc_row_bytes & 15) == 0;
        auto load_group = [&](int kb0, uint32_t (&out)[4]) {
#pragma unroll
          for (int j = 0; j < 4; ++j) out[j] = 0u;
          if (kb0 >= nk_main) return;
          if (!DX) {
            const int n = ps.n0 + r;
            if (n >= p.Wn) return;
            const uint8_t* row = sc_base + (long long)n * sc_row_bytes;
            if (vec_ok && kb0 * 4 + 16 <= sc_row_bytes) {
              const uint4 v = __ldg(reinterpret_cast<const uint4*>(row + kb0 * 4));
              out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (kb0 + j < nk_main) out[j] = __ldg(reinterpret_cast<const uint32_t*>(row + (kb0 + j) * 4));
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) out[j] = (out[j] >> (part * 16)) & 0xFFFFu;
          } else {
            const int k0 = ps.n0 + half * 64 + part * 32;
            if (k0 >= p.Wk) return;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int wn = (kb0 + j) * BK + r;
              if (kb0 + j < nk_main && wn < p.Wn)
                out[j] = __ldg(reinterpret_cast<const unsigned short*>(sc_base + (long long)wn * sc_row_bytes + k0 / 16));
            }
          }
        };
        uint32_t cur[4], nxt[4];
        load_group(0, cur);
        for (int kb0 = 0; kb0 < nk && ok; kb0 += 4) {
          load_group(kb0 + 4, nxt);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int kb = kb0 + j;
            if (kb >= nk) break;
            if (!mbar_wait(&raw_full[stage], phase, p.status, AXB_TIMEOUT_FULL)) {
              ok = false;
              break;
            }
            if (kb < nk_main) {
              uint4 w = *reinterpret_cast<const uint4*>(sRaw + stage * RAW_BYTES + ct * 16);
              uint32_t sc2 = cur[j];                    // two E4M3 bytes: codes 0-15 and 16-31 of this thread
              uint8_t* dst_row = sB + stage * B_BYTES + half * 8192 + r * 128;
              int pos = (part * 4) ^ (r & 7);           // chunk position of this thread's first chunk
              if (DX && half) {
                w = make_uint4(w.z, w.w, w.x, w.y);
                sc2 = ((sc2 >> 8) | (sc2 << 8)) & 0xFFFFu;
                pos ^= 2;
              }
              Lut t = make_lut(e4m3_to_float(sc2 & 0xFF) * g);
              *reinterpret_cast<uint4*>(dst_row + ((pos ^ 0) << 4)) = decode8(w.x, t);
              *reinterpret_cast<uint4*>(dst_row + ((pos ^ 1) << 4)) = decode8(w.y, t);
              t = make_lut(e4m3_to_float(sc2 >> 8) * g);
              *reinterpret_cast<uint4*>(dst_row + ((pos ^ 2) << 4)) = decode8(w.z, t);
              *reinterpret_cast<uint4*>(dst_row + ((pos ^ 3) << 4)) = decode8(w.w, t);
              fence_proxy_async_smem();
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&full_bar[stage]);
            if (++stage == W4_STAGES) {
              stage = 0;
              phase ^= 1;
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) cur[j] = nxt[j];
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps 2..5
    const int lane_group = warp & 3;
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
      for (int sub = 0; sub < 2 && ok; ++sub) {
        Pass ps;
        if (!get_pass(p.blk_expert, n_blocks, num_n, p.E, tile, sub, ps)) continue;
        const int acc = it & 1;
        if (!mbar_wait(&tfull_bar[acc], (it >> 1) & 1, p.status, AXB_TIMEOUT_TMEM_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after();
        for (int h = 0; h <= ps.two; ++h) {
          const long long row = (long long)(ps.blk + h) * BM + lane_group * 32 + lane;
          const uint32_t t_addr = tmem_base + (uint32_t(lane_group * 32) << 16) + acc * 2 * BN + h * BN;
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(t_addr + c * 32, r);
            tmem_ld_wait();
            const int col0 = ps.n0 + c * 32;
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
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[acc]);
        ++it;
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
  p.N = N; p.K = Ka; p.K2 = K2 > 0 ? K2 : 0; p.Wn = Wn; p.Wk = Wk; p.E = E;
  p.C = C; p.ldc = ldc; p.alpha = alpha; p.out_mode = out_mode;
  p.scale = reinterpret_cast<const uint8_t*>(scale); p.pts = pts;
  p.blk_expert = blk_expert; p.n_blocks = n_blocks; p.status = status;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int max_tiles = ((max_blocks + 1) / 2) * ((N + BN - 1) / BN);
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
