// Mixture-of-experts support kernels for sm_100a.
//
//  * nvfp4_dequant     : packed E2M1 nibbles x E4M3 block scales (16 elements) x fp32 per-tensor
//                        scale -> bf16 rows, for the frozen NVFP4 expert weights (storage contract
//                        of src/axolotl/integrations/kernels/libs/scattermoe_lora/dequant_grouped.py:63-111).
//  * ep_gather_rows    : expert-parallel DISPATCH. Every destination rank pulls the token rows
//                        routed to its experts straight out of the source ranks' symmetric
//                        activation buffers with peer loads over NVLink (row list: source rank +
//                        source row), writing them expert-sorted into a local buffer.
//  * ep_scatter_add    : expert-parallel COMBINE. Expert outputs are multiplied by their routing
//                        weight and reduce-added (bf16x2 atomics over NVLink) into the source
//                        rank's output buffer at the token's row.
//  * peer_put_i32      : routing metadata exchange (plain peer stores).
// Together they replace DeepEP's dispatch / combine + host barrier of the reference
// (src/axolotl/integrations/expert_parallel/experts_fn.py:185-342).
#include "axb_common.cuh"

namespace {

// bf16 bit patterns of the 8 E2M1 magnitudes {0, .5, 1, 1.5, 2, 3, 4, 6}, 16 bits each, held in two
// 64-bit registers: a lookup is a shift (no memory access, no divergence).
constexpr unsigned long long kE2M1Lo = 0x3fc03f803f000000ull;  // 1.5, 1.0, 0.5, 0.0
constexpr unsigned long long kE2M1Hi = 0x40c0408040404000ull;  // 6.0, 4.0, 3.0, 2.0

AXB_DEVICE float e2m1_to_float(uint32_t code) {
  const unsigned long long tbl = (code & 4) ? kE2M1Hi : kE2M1Lo;
  const uint32_t bits = (uint32_t)(tbl >> ((code & 3) * 16)) & 0xFFFFu;
  return __uint_as_float((bits | ((code & 8) << 12)) << 16);
}

AXB_DEVICE float e4m3_to_float(uint8_t v) {
  const uint32_t sign = (v >> 7) & 1, exp = (v >> 3) & 0xF, man = v & 7;
  float f;
  if (exp == 0) f = ldexpf((float)man, -9);                 // subnormal: man * 2^-3 * 2^-6
  else if (exp == 15 && man == 7) f = __int_as_float(0x7fc00000);
  else f = __uint_as_float(((exp + 120u) << 23) | (man << 20));
  return sign ? -f : f;
}

// One thread per 16 bytes of packed codes (32 values = two 16-element scale blocks): 16-byte
// loads, four 16-byte stores; a warp reads 512 contiguous bytes and writes 2 KB contiguous.
__global__ void nvfp4_dequant_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ scale,
                                     const float* __restrict__ pts, __nv_bfloat16* __restrict__ out,
                                     long long n_blocks, long long blocks_per_pts,
                                     const int* __restrict__ active) {
  const long long n_pairs = n_blocks >> 1;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < n_pairs;
       t += (long long)gridDim.x * blockDim.x) {
    const long long b = t * 2;
    const long long mat = b / blocks_per_pts;
    if (active && active[mat] == 0) continue;   // selective dequant: no row is routed to this expert
    const float g = pts[mat];
    const unsigned short sc = *reinterpret_cast<const unsigned short*>(scale + b);
    const float s0 = e4m3_to_float(sc & 0xFF) * g, s1 = e4m3_to_float(sc >> 8) * g;
    const uint4 packed = *reinterpret_cast<const uint4*>(q + b * 8);
    const uint32_t w[4] = {packed.x, packed.y, packed.z, packed.w};
    uint32_t o[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float s = i < 2 ? s0 : s1;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t byte = (w[i] >> (8 * j)) & 0xFF;
        o[i * 4 + j] = pack_bf16x2(e2m1_to_float(byte & 0xF) * s, e2m1_to_float(byte >> 4) * s);
      }
    }
    uint4* dst = reinterpret_cast<uint4*>(out + b * 16);
#pragma unroll
    for (int i = 0; i < 4; ++i) dst[i] = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
  }
  // odd trailing block (K/16 odd for a single row) is handled by the last thread
  if ((n_blocks & 1) && blockIdx.x == 0 && threadIdx.x == 0) {
    const long long b = n_blocks - 1;
    const float s = e4m3_to_float(scale[b]) * pts[b / blocks_per_pts];
    for (int i = 0; i < 8; ++i) {
      const uint32_t byte = q[b * 8 + i];
      out[b * 16 + 2 * i] = __float2bfloat16(e2m1_to_float(byte & 0xF) * s);
      out[b * 16 + 2 * i + 1] = __float2bfloat16(e2m1_to_float(byte >> 4) * s);
    }
  }
}

// Local dispatch: out[r, :] = row_token[r] >= 0 ? scale[r] * x[row_token[r], :] : 0 for every row of
// the padded expert-sorted layout (one warp per row; pad rows are written as zeros).
__global__ void moe_dispatch_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ row_token,
                                         const float* __restrict__ row_scale, __nv_bfloat16* __restrict__ out,
                                         long long n_rows, int width) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r = w; r < n_rows; r += n_warps) {
    const int tok = row_token[r];
    __nv_bfloat16* d = out + r * width;
    if (tok < 0) {
      for (int c = lane * 8; c < width; c += 256) *reinterpret_cast<uint4*>(d + c) = make_uint4(0, 0, 0, 0);
      continue;
    }
    const __nv_bfloat16* s = x + (long long)tok * width;
    const float g = row_scale ? row_scale[r] : 1.f;
    for (int c = lane * 8; c < width; c += 256) {
      uint4 v = *reinterpret_cast<const uint4*>(s + c);
      if (row_scale) {
        uint32_t in[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_bf16x2(in[e]);
          in[e] = pack_bf16x2(f.x * g, f.y * g);
        }
        v = make_uint4(in[0], in[1], in[2], in[3]);
      }
      *reinterpret_cast<uint4*>(d + c) = v;
    }
  }
}

// Local combine: out[t, :] = sum_j w[t, j] * ys[slot_row[t, j], :] (fp32 accumulation, no atomics).
template <int TOPK_MAX>
__global__ void moe_combine_rows_kernel(const __nv_bfloat16* __restrict__ ys, const int* __restrict__ slot_row,
                                        const float* __restrict__ w, __nv_bfloat16* __restrict__ out,
                                        long long n_tokens, int k, int width) {
  const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long t = wid; t < n_tokens; t += n_warps) {
    for (int c = lane * 8; c < width; c += 256) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < k; ++j) {
        const int r = slot_row[t * k + j];
        const float g = w ? w[t * k + j] : 1.f;
        const uint4 v = *reinterpret_cast<const uint4*>(ys + (long long)r * width + c);
        const uint32_t in[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_bf16x2(in[e]);
          acc[2 * e] += g * f.x;
          acc[2 * e + 1] += g * f.y;
        }
      }
      *reinterpret_cast<uint4*>(out + t * width + c) =
          make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                     pack_bf16x2(acc[6], acc[7]));
    }
  }
}

// dw[t, j] = <dy[t, :], ys[slot_row[t, j], :]>  (gradient of the routing weights; one warp per slot)
__global__ void moe_combine_dw_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ ys,
                                      const int* __restrict__ slot_row, float* __restrict__ dw, long long n_slots,
                                      int k, int width) {
  const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long sl = wid; sl < n_slots; sl += n_warps) {
    const __nv_bfloat16* a = dy + (sl / k) * width;
    const __nv_bfloat16* b = ys + (long long)slot_row[sl] * width;
    float acc = 0.f;
    for (int c = lane * 8; c < width; c += 256) {
      const uint4 va = *reinterpret_cast<const uint4*>(a + c), vb = *reinterpret_cast<const uint4*>(b + c);
      const uint32_t ia[4] = {va.x, va.y, va.z, va.w}, ib[4] = {vb.x, vb.y, vb.z, vb.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 fa = unpack_bf16x2(ia[e]), fb = unpack_bf16x2(ib[e]);
        acc += fa.x * fb.x + fa.y * fb.y;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) dw[sl] = acc;
  }
}

struct PeerPtrs8 {
  unsigned long long p[8];
};

// out[i, :] = scale(i) * src_rank(i).buffer[src_row(i), :]   (one warp per row, 16-byte vectors).
// src_rank(i) < 0 marks a pad row of the expert-sorted layout: it is written as zeros.
// Optionally dot_out[i] = <unscaled gathered row, dot_with[i, :]> (gradient of the routing weight).
__global__ void ep_gather_rows_kernel(PeerPtrs8 src, const int* __restrict__ src_rank,
                                      const int* __restrict__ src_row, const float* __restrict__ scale,
                                      const __nv_bfloat16* __restrict__ dot_with, float* __restrict__ dot_out,
                                      __nv_bfloat16* __restrict__ out, long long n_rows, int width, long long src_ld,
                                      const int* __restrict__ blocks_in_use) {
  if (blocks_in_use) n_rows = min(n_rows, (long long)(*blocks_in_use) * 128);   // rows beyond the used blocks are never read
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long i = w; i < n_rows; i += n_warps) {
    const int rk = src_rank[i];
    if (rk < 0) {
      for (int c = lane * 8; c < width; c += 256)
        *reinterpret_cast<uint4*>(out + i * width + c) = make_uint4(0, 0, 0, 0);
      if (dot_out && lane == 0) dot_out[i] = 0.f;
      continue;
    }
    const __nv_bfloat16* s = reinterpret_cast<const __nv_bfloat16*>(src.p[rk]) + (long long)src_row[i] * src_ld;
    const float g = scale ? scale[i] : 1.f;
    float acc = 0.f;
    for (int c = lane * 8; c < width; c += 256) {
      uint4 v = *reinterpret_cast<const uint4*>(s + c);
      if (dot_with) {
        const uint4 d = *reinterpret_cast<const uint4*>(dot_with + i * width + c);
        const uint32_t a[4] = {v.x, v.y, v.z, v.w}, b[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 fa = unpack_bf16x2(a[e]), fb = unpack_bf16x2(b[e]);
          acc += fa.x * fb.x + fa.y * fb.y;
        }
      }
      if (scale) {
        uint32_t in[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_bf16x2(in[e]);
          in[e] = pack_bf16x2(f.x * g, f.y * g);
        }
        v = make_uint4(in[0], in[1], in[2], in[3]);
      }
      *reinterpret_cast<uint4*>(out + i * width + c) = v;
    }
    if (dot_out) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lane == 0) dot_out[i] = acc;
    }
  }
}

// Deduplicated dispatch: a token with several slots on this rank crosses NVLink once.
// staging[r][row][:] = rank r's buffer[row][:] for every (r != self, row) with need[r*T + row] set.
__global__ void ep_stage_rows_kernel(PeerPtrs8 src, const unsigned char* __restrict__ need,
                                     __nv_bfloat16* __restrict__ staging, int world, int self, long long T,
                                     int width) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const long long items = (long long)world * T;
  for (long long i = w; i < items; i += n_warps) {
    const int r = (int)(i / T);
    if (r == self || !need[i]) continue;
    const long long row = i - (long long)r * T;
    const __nv_bfloat16* s = reinterpret_cast<const __nv_bfloat16*>(src.p[r]) + row * width;
    __nv_bfloat16* d = staging + i * width;
    // all loads of a batch are issued before the first store: up to 8 x 16 B per lane (4 KB per warp)
    // in flight over NVLink instead of one vector
    for (int c0 = lane * 8; c0 < width; c0 += 256 * 8) {
      uint4 v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (c0 + k * 256 < width) v[k] = *reinterpret_cast<const uint4*>(s + c0 + k * 256);
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (c0 + k * 256 < width) *reinterpret_cast<uint4*>(d + c0 + k * 256) = v[k];
    }
  }
}

// Deduplicated combine: every expert rank first sums its slots of a token locally into
// partial[source rank][row]; the source then adds one partial row per contributing rank:
// y[row][:] += sum over r != self with sent[r*T + row] of rank r's partial[self*T + row][:].
__global__ void ep_reduce_rows_kernel(PeerPtrs8 part, const unsigned char* __restrict__ sent,
                                      __nv_bfloat16* __restrict__ y, int world, int self, long long T, int width) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long row = w; row < T; row += n_warps) {
    unsigned mask = 0;
    for (int r = 0; r < world; ++r)
      if (r != self && sent[(long long)r * T + row]) mask |= 1u << r;
    if (!mask) continue;
    for (int c = lane * 8; c < width; c += 256) {
      float acc[8];
      {
        const uint4 v = *reinterpret_cast<const uint4*>(y + row * width + c);
        const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), cc = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
        acc[0] = a.x; acc[1] = a.y; acc[2] = b.x; acc[3] = b.y; acc[4] = cc.x; acc[5] = cc.y; acc[6] = d.x; acc[7] = d.y;
      }
      // peer loads first (independent, all in flight together), sums afterwards
      uint4 pv[8];
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < world && ((mask >> r) & 1u))
          pv[r] = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(part.p[r]) +
                                                  ((long long)self * T + row) * width + c);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (!(r < world && ((mask >> r) & 1u))) continue;
        const uint4 v = pv[r];
        const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), cc = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
        acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += cc.x; acc[5] += cc.y; acc[6] += d.x; acc[7] += d.y;
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(y + row * width + c) = o;
    }
  }
}

// dst_rank(i).buffer[dst_row(i), :] += weight(i) * rows[i, :]
__global__ void ep_scatter_add_kernel(PeerPtrs8 dst, const int* __restrict__ dst_rank,
                                      const int* __restrict__ dst_row, const float* __restrict__ weight,
                                      const __nv_bfloat16* __restrict__ rows, long long n_rows, int width,
                                      long long dst_ld) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long i = w; i < n_rows; i += n_warps) {
    if (dst_rank[i] < 0) continue;   // pad row of the expert-sorted layout
    const float g = weight ? weight[i] : 1.f;
    __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(dst.p[dst_rank[i]]) + (long long)dst_row[i] * dst_ld;
    for (int c = lane * 8; c < width; c += 256) {
      const uint4 v = *reinterpret_cast<const uint4*>(rows + i * width + c);
      const uint32_t in[4] = {v.x, v.y, v.z, v.w};
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf16x2(in[e]);
        o[e] = pack_bf16x2(f.x * g, f.y * g);
      }
      asm volatile("red.relaxed.sys.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(d + c), "r"(o[0]),
                   "r"(o[1]), "r"(o[2]), "r"(o[3])
                   : "memory");
    }
  }
}

__global__ void peer_put_i32_kernel(int* __restrict__ dst, const int* __restrict__ src, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dst[i] = src[i];
}

// Routing tables of every rank into one local array: dst[r * n + i] = peer r's src[i] (plain peer loads).
__global__ void ep_gather_tables_kernel(PeerPtrs8 src, int world, long long n, int* __restrict__ dst) {
  const long long total = (long long)world * n;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / n);
    dst[i] = reinterpret_cast<const int*>(src.p[r])[i - (long long)r * n];
  }
}

// Per-slot scalars back to the rank that routed the slot: peer src_rank[i] gets vals[i] at slot src_slot[i]
// (rows with src_rank < 0 are padding). Plain peer stores; the caller's barrier publishes them.
__global__ void ep_put_scalars_kernel(PeerPtrs8 dst, const int* __restrict__ src_rank, const int* __restrict__ src_slot,
                                      const float* __restrict__ vals, long long n, long long slots) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int r = src_rank[i], sl = src_slot[i];
    if (r < 0 || sl < 0 || sl >= slots) continue;
    reinterpret_cast<float*>(dst.p[r])[sl] = vals[i];
  }
}

int fill8(PeerPtrs8& d, const unsigned long long* s, int world) {
  if (world < 1 || world > 8) return -2;
  for (int i = 0; i < 8; ++i) d.p[i] = i < world ? s[i] : 0ull;
  return 0;
}
}  // namespace

#define ST(s) reinterpret_cast<cudaStream_t>(s)

// q: [rows, cols/2] uint8, scale: [rows, cols/16] e4m3 bytes, pts: device fp32 scalar -> out [rows, cols] bf16
extern "C" int axb_nvfp4_dequant(const void* q, const void* scale, const float* pts, void* out, long long rows,
                                 long long cols, void* stream) {
  if (cols % 16) return -2;
  const long long nb = rows * (cols / 16);
  if (nb <= 0) return 0;
  int grid = (int)((nb / 2 + 255) / 256 > 148 * 16 ? 148 * 16 : (nb / 2 + 255) / 256);
  if (grid < 1) grid = 1;
  nvfp4_dequant_kernel<<<grid, 256, 0, ST(stream)>>>((const uint8_t*)q, (const uint8_t*)scale, pts,
                                                     (__nv_bfloat16*)out, nb, nb, nullptr);
  return (int)cudaGetLastError();
}

// batch of matrices (expert stacks): q [batch, rows, cols/2], scale [batch, rows, cols/16],
// pts [batch] fp32 -> out [batch, rows, cols] bf16, one launch. ``active`` (int32 [batch], optional):
// matrices whose entry is 0 are skipped and their output left untouched (experts without routed
// rows: what a decode step or a small batch saves).
extern "C" int axb_nvfp4_dequant_batched(const void* q, const void* scale, const float* pts, void* out,
                                         long long batch, long long rows, long long cols, const int* active,
                                         void* stream) {
  if (cols % 16) return -2;
  const long long per = rows * (cols / 16);
  const long long nb = batch * per;
  if (nb <= 0) return 0;
  int grid = (int)((nb / 2 + 255) / 256 > 148 * 16 ? 148 * 16 : (nb / 2 + 255) / 256);
  if (grid < 1) grid = 1;
  nvfp4_dequant_kernel<<<grid, 256, 0, ST(stream)>>>((const uint8_t*)q, (const uint8_t*)scale, pts,
                                                     (__nv_bfloat16*)out, nb, per, active);
  return (int)cudaGetLastError();
}

static int rows_grid(long long n_rows) {
  const long long want = (n_rows + 7) / 8;   // 8 warps (rows) per 256-thread block
  return (int)(want > 148 * 8 ? 148 * 8 : (want < 1 ? 1 : want));
}

// out [n_rows, width] bf16; row_token int32 [n_rows] (-1 = zero row); row_scale fp32 [n_rows] or NULL
extern "C" int axb_moe_dispatch_rows(const void* x, const int* row_token, const float* row_scale, void* out,
                                     long long n_rows, int width, void* stream) {
  if (width % 8) return -2;
  if (n_rows <= 0) return 0;
  moe_dispatch_rows_kernel<<<rows_grid(n_rows), 256, 0, ST(stream)>>>(
      (const __nv_bfloat16*)x, row_token, row_scale, (__nv_bfloat16*)out, n_rows, width);
  return (int)cudaGetLastError();
}

// out [n_tokens, width] = sum_j w[t, j] * ys[slot_row[t, j]]; w fp32 [n_tokens, k] or NULL (= 1)
extern "C" int axb_moe_combine_rows(const void* ys, const int* slot_row, const float* w, void* out,
                                    long long n_tokens, int k, int width, void* stream) {
  if (width % 8) return -2;
  if (n_tokens <= 0) return 0;
  moe_combine_rows_kernel<16><<<rows_grid(n_tokens), 256, 0, ST(stream)>>>(
      (const __nv_bfloat16*)ys, slot_row, w, (__nv_bfloat16*)out, n_tokens, k, width);
  return (int)cudaGetLastError();
}

extern "C" int axb_moe_combine_dw(const void* dy, const void* ys, const int* slot_row, float* dw,
                                  long long n_slots, int k, int width, void* stream) {
  if (width % 8) return -2;
  if (n_slots <= 0) return 0;
  moe_combine_dw_kernel<<<rows_grid(n_slots), 256, 0, ST(stream)>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)ys, slot_row, dw, n_slots, k, width);
  return (int)cudaGetLastError();
}

// src_rank[i] < 0 => zero row; scale (fp32 per row) / dot_with (bf16 [n_rows, width]) + dot_out are optional
extern "C" int axb_ep_gather_rows(const unsigned long long* src_ptrs, int world, const int* src_rank,
                                  const int* src_row, const float* scale, const void* dot_with, float* dot_out,
                                  void* out, long long n_rows, int width, long long src_ld, void* stream) {
  if (n_rows <= 0) return 0;
  if (width % 8 || src_ld % 8) return -2;
  PeerPtrs8 p;
  if (fill8(p, src_ptrs, world)) return -2;
  int grid = (int)((n_rows + 7) / 8 > 148 * 8 ? 148 * 8 : (n_rows + 7) / 8);
  ep_gather_rows_kernel<<<grid, 256, 0, ST(stream)>>>(p, src_rank, src_row, scale, (const __nv_bfloat16*)dot_with,
                                                      dot_out, (__nv_bfloat16*)out, n_rows, width, src_ld, nullptr);
  return (int)cudaGetLastError();
}
// the same over the first *blocks_in_use * 128 rows only (device-side count of the capacity-bounded plan)
extern "C" int axb_ep_gather_rows_n(const unsigned long long* src_ptrs, int world, const int* src_rank,
                                    const int* src_row, const float* scale, const void* dot_with, float* dot_out,
                                    void* out, long long n_rows, int width, long long src_ld, const int* blocks_in_use,
                                    void* stream) {
  if (n_rows <= 0) return 0;
  if (width % 8 || src_ld % 8) return -2;
  PeerPtrs8 p;
  if (fill8(p, src_ptrs, world)) return -2;
  int grid = (int)((n_rows + 7) / 8 > 148 * 8 ? 148 * 8 : (n_rows + 7) / 8);
  ep_gather_rows_kernel<<<grid, 256, 0, ST(stream)>>>(p, src_rank, src_row, scale, (const __nv_bfloat16*)dot_with,
                                                      dot_out, (__nv_bfloat16*)out, n_rows, width, src_ld, blocks_in_use);
  return (int)cudaGetLastError();
}

extern "C" int axb_ep_scatter_add(const unsigned long long* dst_ptrs, int world, const int* dst_rank,
                                  const int* dst_row, const float* weight, const void* rows, long long n_rows,
                                  int width, long long dst_ld, void* stream) {
  if (n_rows <= 0) return 0;
  if (width % 8 || dst_ld % 8) return -2;
  PeerPtrs8 p;
  if (fill8(p, dst_ptrs, world)) return -2;
  int grid = (int)((n_rows + 7) / 8 > 148 * 8 ? 148 * 8 : (n_rows + 7) / 8);
  ep_scatter_add_kernel<<<grid, 256, 0, ST(stream)>>>(p, dst_rank, dst_row, weight, (const __nv_bfloat16*)rows, n_rows,
                                                      width, dst_ld);
  return (int)cudaGetLastError();
}

extern "C" int axb_ep_stage_rows(const unsigned long long* src_ptrs, int world, int self, const void* need,
                                 void* staging, long long T, int width, void* stream) {
  if (T <= 0) return 0;
  if (width % 8) return -2;
  PeerPtrs8 p;
  if (fill8(p, src_ptrs, world)) return -2;
  const long long items = (long long)world * T;
  int grid = (int)((items + 7) / 8 > 148 * 8 ? 148 * 8 : (items + 7) / 8);
  ep_stage_rows_kernel<<<grid, 256, 0, ST(stream)>>>(p, (const unsigned char*)need, (__nv_bfloat16*)staging, world,
                                                     self, T, width);
  return (int)cudaGetLastError();
}

extern "C" int axb_ep_reduce_rows(const unsigned long long* part_ptrs, int world, int self, const void* sent,
                                  void* y, long long T, int width, void* stream) {
  if (T <= 0) return 0;
  if (width % 8) return -2;
  PeerPtrs8 p;
  if (fill8(p, part_ptrs, world)) return -2;
  int grid = (int)((T + 7) / 8 > 148 * 8 ? 148 * 8 : (T + 7) / 8);
  ep_reduce_rows_kernel<<<grid, 256, 0, ST(stream)>>>(p, (const unsigned char*)sent, (__nv_bfloat16*)y, world, self,
                                                      T, width);
  return (int)cudaGetLastError();
}

extern "C" int axb_ep_gather_tables(const unsigned long long* src_ptrs, int world, long long n, void* dst, void* stream) {
  PeerPtrs8 s;
  if (fill8(s, src_ptrs, world)) return -2;
  if (n <= 0) return 0;
  const long long total = (long long)world * n;
  int grid = (int)((total + 255) / 256 > 148 * 8 ? 148 * 8 : (total + 255) / 256);
  ep_gather_tables_kernel<<<grid, 256, 0, ST(stream)>>>(s, world, n, (int*)dst);
  return (int)cudaGetLastError();
}

extern "C" int axb_ep_put_scalars(const unsigned long long* dst_ptrs, int world, const void* src_rank,
                                  const void* src_slot, const void* vals, long long n, long long slots, void* stream) {
  PeerPtrs8 d;
  if (fill8(d, dst_ptrs, world)) return -2;
  if (n <= 0) return 0;
  int grid = (int)((n + 255) / 256 > 148 * 8 ? 148 * 8 : (n + 255) / 256);
  ep_put_scalars_kernel<<<grid, 256, 0, ST(stream)>>>(d, (const int*)src_rank, (const int*)src_slot, (const float*)vals, n, slots);
  return (int)cudaGetLastError();
}

extern "C" int axb_peer_put_i32(void* dst, const void* src, long long n, void* stream) {
  if (n <= 0) return 0;
  int grid = (int)((n + 255) / 256 > 148 * 4 ? 148 * 4 : (n + 255) / 256);
  peer_put_i32_kernel<<<grid, 256, 0, ST(stream)>>>((int*)dst, (const int*)src, n);
  return (int)cudaGetLastError();
}
