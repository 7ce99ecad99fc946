// Common sm_100a device helpers: mbarrier, TMA, tcgen05/TMEM wrappers with bounded waits.
//
// Every wait in this library is bounded: when the budget runs out the waiter records a
// status code in a global status word and returns false, so the caller can unwind (free
// TMEM, leave the kernel) and the host can raise a Python exception instead of hanging
// the GPU.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda.h>
#include <stdint.h>

#define AXB_DEVICE __device__ __forceinline__

// status codes written to the status word (0 = ok)
enum AxbStatus : int {
  AXB_OK = 0,
  AXB_TIMEOUT_FULL = 1,     // consumer waited for a TMA stage that never arrived
  AXB_TIMEOUT_EMPTY = 2,    // producer waited for a stage that was never released
  AXB_TIMEOUT_TMEM_FULL = 3,
  AXB_TIMEOUT_TMEM_EMPTY = 4,
  AXB_TIMEOUT_PEER_FLAG = 5,  // a flag written by another GPU / CTA never arrived
  AXB_BAD_ARGUMENT = 6,
  AXB_TIMEOUT_GENERIC = 7,
};

// Bounds-check build (-DAXB_BOUNDS_CHECK, linked as libaxb200_checked.so): every data-dependent index that a
// kernel reads from device memory (token ids, labels, expert ids, document tiles) is compared with its
// limit before the access; the first violation is recorded (site, index, limit) in a device record that
// the host reads through axb_bounds_fetch, and the access is skipped. The regular build compiles the
// checks away.
enum AxbBoundsSite : int {
  AXB_SITE_EMBED_ID = 1,
  AXB_SITE_EMBED_GRAD_ID = 2,
  AXB_SITE_CE_LABEL = 3,
  AXB_SITE_GROUPED_EXPERT = 4,
  AXB_SITE_W4A16_EXPERT = 5,
  AXB_SITE_ATTN_TILE = 6,
  AXB_SITE_DISPATCH_TOKEN = 7,
};
#ifdef AXB_BOUNDS_CHECK
extern __device__ unsigned long long axb_bounds_record[4];   // site, index, limit, count (bounds_check.cu)
AXB_DEVICE bool axb_index_ok(int site, long long idx, long long limit) {
  if (idx >= 0 && idx < limit) return true;
  atomicAdd(&axb_bounds_record[3], 1ull);
  if (atomicCAS(&axb_bounds_record[0], 0ull, (unsigned long long)site) == 0ull) {
    axb_bounds_record[1] = (unsigned long long)idx;
    axb_bounds_record[2] = (unsigned long long)limit;
  }
  return false;
}
#define AXB_INDEX_OK(site, idx, limit) axb_index_ok((site), (long long)(idx), (long long)(limit))
#else
#define AXB_INDEX_OK(site, idx, limit) true
#endif

// wait budget in nanoseconds of %globaltimer (2 s: far above any legitimate wait)
#ifndef AXB_WAIT_BUDGET_NS
#define AXB_WAIT_BUDGET_NS 2000000000ull
#endif

AXB_DEVICE uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

AXB_DEVICE uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

AXB_DEVICE bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred P1;\n\t"
      "elect.sync _|P1, 0xFFFFFFFF;\n\t"
      "selp.b32 %0, 1, 0, P1;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ------------------------------------------------------------------ mbarrier
AXB_DEVICE void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
AXB_DEVICE void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
AXB_DEVICE void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
AXB_DEVICE void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
AXB_DEVICE bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait. Returns false (after writing `code` to *status) when the budget ran out.
AXB_DEVICE bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0x3FF) == 0) {
      if (global_timer_ns() - t0 > AXB_WAIT_BUDGET_NS) {
        if (status) atomicCAS(status, 0, code);
        return false;
      }
    }
  }
  return true;
}

// Non-suspending variant (mbarrier.test_wait in a spin loop). Used by the CTA-pair kernels:
// a suspended try_wait was observed not to be woken promptly by arrivals that come from the
// partner CTA / a cta_group::2 commit, which serialised the pipeline at one stage per time-out.
AXB_DEVICE bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
AXB_DEVICE bool mbar_wait_spin(uint64_t* bar, uint32_t parity, int* status, int code) {
  if (mbar_test_wait(bar, parity)) return true;
  uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_test_wait(bar, parity)) {
    if ((++spins & 0xFFF) == 0) {
      if (global_timer_ns() - t0 > AXB_WAIT_BUDGET_NS) {
        if (status) atomicCAS(status, 0, code);
        return false;
      }
    }
  }
  return true;
}

// ------------------------------------------------------------------ TMA (no multicast anywhere)
AXB_DEVICE void tma_load_2d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int c0,
                            int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
      "%4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)),
        "r"(c0), "r"(c1)
      : "memory");
}
AXB_DEVICE void tma_load_3d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int c0,
                            int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
      "%4, %5}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)),
        "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
AXB_DEVICE void tma_prefetch_desc(const CUtensorMap* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
// plain (untiled) bulk copy global -> shared, 16-byte aligned addresses and size
AXB_DEVICE void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes),
        "r"(smem_u32(bar))
      : "memory");
}
// tile store shared -> global (bulk async group of the issuing thread); out-of-range rows / columns
// of the box are clipped by the tensor map
AXB_DEVICE void tma_store_2d(const CUtensorMap* tmap, const void* smem_src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               :
               : "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1)
               : "memory");
}
AXB_DEVICE void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all but the newest N bulk groups of this thread have finished READING shared memory
template <int N>
AXB_DEVICE void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
AXB_DEVICE void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
AXB_DEVICE void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ------------------------------------------------------------------ tcgen05 / TMEM
AXB_DEVICE void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
AXB_DEVICE void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
AXB_DEVICE void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
AXB_DEVICE void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
AXB_DEVICE void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]; kind::f16 covers bf16/fp16 inputs, fp32 accumulate.
AXB_DEVICE void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                         uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on an mbarrier once all previously issued tcgen05.mma of this thread have completed
AXB_DEVICE void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
AXB_DEVICE void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
AXB_DEVICE void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32 lanes x 32 consecutive fp32 columns: thread t of the warp receives row (lane base + t).
AXB_DEVICE void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
AXB_DEVICE void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// ------------------------------------------------------------------ CTA pairs (cta_group::2)
AXB_DEVICE uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
AXB_DEVICE void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `smem_addr` (a shared::cta address of this CTA) inside CTA `rank`
AXB_DEVICE uint32_t mapa_u32(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
AXB_DEVICE void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
AXB_DEVICE void mbar_expect_tx_cluster(uint32_t cluster_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr),
               "r"(bytes)
               : "memory");
}
// TMA tile load issued by one CTA of a pair; completion bytes are credited to the mbarrier at
// cluster address `bar_cluster_addr` (the leader CTA's barrier). No multicast.
AXB_DEVICE void tma_load_2d_pair(void* smem_dst, const CUtensorMap* tmap, uint32_t bar_cluster_addr, int c0,
                                 int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
AXB_DEVICE void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
AXB_DEVICE void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
AXB_DEVICE void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// one instruction drives the tensor cores of both SMs of the pair: D[256 x N] += A[256 x 16] B[N x 16]^T
AXB_DEVICE void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                              uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive (once the pair's MMAs issued so far retire) on the mbarrier at cluster address `addr`
AXB_DEVICE void umma_commit_pair_addr(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}
// same, one instruction for both CTAs of the pair (mask 0b11) -- tcgen05.commit's own multicast
AXB_DEVICE void umma_commit_pair_mc(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"((uint16_t)3)
      : "memory");
}
// ... on the barrier at the same shared-memory offset in both CTAs of the pair (issued by rank 0)
AXB_DEVICE void umma_commit_pair_both(uint64_t* bar) {
  const uint32_t a = smem_u32(bar);
  umma_commit_pair_addr(mapa_u32(a, 0));
  umma_commit_pair_addr(mapa_u32(a, 1));
}

// Shared-memory matrix descriptor for tcgen05.mma, 128-byte swizzle.
//   K-major tile (rows of 64 bf16 = 128 B, 8-row atoms of 1024 B): lbo unused, sbo = 1024.
//   MN-major tile (64 contiguous MN elements per k row, 8 k rows per 1024 B atom):
//     lbo = byte stride between 64-element MN chunks, sbo = byte stride between 8-row k groups.
AXB_DEVICE uint64_t make_smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);              // bits [0,14)
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;     // bits [16,30)
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;     // bits [32,46)
  d |= static_cast<uint64_t>(1) << 46;                             // descriptor version (Blackwell)
  d |= static_cast<uint64_t>(2) << 61;                             // SWIZZLE_128B
  return d;
}

// Instruction descriptor, kind::f16, bf16 inputs, fp32 accumulator.
AXB_DEVICE constexpr uint32_t make_idesc_bf16(int m, int n, int a_mn_major, int b_mn_major) {
  return (1u << 4)                       // D format: f32
         | (1u << 7)                     // A format: bf16
         | (1u << 10)                    // B format: bf16
         | (uint32_t(a_mn_major) << 15)  // A major
         | (uint32_t(b_mn_major) << 16)  // B major
         | (uint32_t(n >> 3) << 17)      // N / 8
         | (uint32_t(m >> 4) << 24);     // M / 16
}

AXB_DEVICE uint32_t pack_bf16x2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
AXB_DEVICE float2 unpack_bf16x2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}

// ------------------------------------------------------------------ host helpers
#include <cstdio>
#include <mutex>
typedef CUresult (*AxbEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                     const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                     const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline AxbEncodeTiledFn axb_get_encode_fn() {
  static AxbEncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<AxbEncodeTiledFn>(p);
  });
  return fn;
}
// 2-D bf16 row-major [rows, cols] with leading stride ld (elements); box = [box_rows, box_cols].
// Returns 0 on success.
inline int axb_make_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                            uint64_t ld_elems, uint32_t box_rows, uint32_t box_cols,
                            int elem_bytes = 2, bool swizzle128 = true, bool swizzle64 = false) {
  AxbEncodeTiledFn fn = axb_get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld_elems * (uint64_t)elem_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                             : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = CUDA_SUCCESS;
  for (int attempt = 0; attempt < 2; ++attempt) {
    r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE,
           swizzle64 ? CU_TENSOR_MAP_SWIZZLE_64B
                     : (swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE),
           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_ERROR_INVALID_CONTEXT) break;
    // A thread that has made no runtime call yet (e.g. an autograd worker) has no current
    // driver context: bind the primary context of the runtime's current device and retry.
    cudaFree(nullptr);
  }
  if (r != CUDA_SUCCESS)
    fprintf(stderr,
            "axb_make_tmap_2d failed: CUresult %d base %p rows %llu cols %llu ld %llu box [%u, %u] "
            "elem_bytes %d\n",
            (int)r, base, (unsigned long long)rows, (unsigned long long)cols,
            (unsigned long long)ld_elems, box_rows, box_cols, elem_bytes);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

// 3-D map over a batch of row-major matrices [batch, rows, cols] (leading dimension ld_elems,
// matrices batch_stride_elems apart); a box is [1, box_rows, box_cols], so its shared-memory
// image equals the 2-D one and a box never crosses into the next matrix of the batch.
inline int axb_make_tmap_3d(CUtensorMap* out, const void* base, uint64_t batch, uint64_t rows,
                            uint64_t cols, uint64_t ld_elems, uint64_t batch_stride_elems,
                            uint32_t box_rows, uint32_t box_cols) {
  AxbEncodeTiledFn fn = axb_get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[3] = {cols, rows, batch};
  cuuint64_t strides[2] = {ld_elems * 2ull, batch_stride_elems * 2ull};
  cuuint32_t box[3] = {box_cols, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = CUDA_SUCCESS;
  for (int attempt = 0; attempt < 2; ++attempt) {
    r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box,
           estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_ERROR_INVALID_CONTEXT) break;
    cudaFree(nullptr);  // bind the primary context on threads that have none yet
  }
  if (r != CUDA_SUCCESS)
    fprintf(stderr,
            "axb_make_tmap_3d failed: CUresult %d base %p batch %llu rows %llu cols %llu ld %llu "
            "stride %llu box [%u, %u]\n",
            (int)r, base, (unsigned long long)batch, (unsigned long long)rows,
            (unsigned long long)cols, (unsigned long long)ld_elems,
            (unsigned long long)batch_stride_elems, box_rows, box_cols);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}
