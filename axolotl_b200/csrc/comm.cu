// Cross-GPU kernels over NVLink peer memory / NVSwitch multicast (one process per GPU; buffers
// come from a symmetric allocation whose peer addresses are mapped into every process).
//
//  * axb_peer_barrier        : flag barrier over the ranks' signal pads, bounded waits.
//  * axb_rs_adamw_ag         : ONE kernel that reduce-scatters the flat fp32 gradient
//                              (multimem.ld_reduce through the switch, or plain peer loads),
//                              derives the global gradient norm, applies clip + AdamW to the
//                              slice this rank owns and publishes the updated fp32 master and
//                              bf16 compute copy to every rank (multimem.st or peer stores).
//                              It replaces NCCL reduce-scatter + clip_grad_norm_ + fused AdamW +
//                              the next step's parameter all-gather of the reference's FSDP2 path.
//  * axb_peer_allreduce_f32  : small one-shot all-reduce (scalars, router statistics).
//
// No TMA multicast is used anywhere; remote data moves with ld/st/multimem issued by threads.
#include <cooperative_groups.h>

#include "axb_common.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int MAX_WORLD = 16;
// signal pad layout (uint32 slots): [channel][src_rank]; channel c starts at word 512 + 16*c
constexpr int PAD_BASE_WORD = 512;

struct PeerPtrs {
  unsigned long long p[MAX_WORLD];
};

AXB_DEVICE void st_release_sys(unsigned int* addr, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
AXB_DEVICE unsigned int ld_acquire_sys(const unsigned int* addr) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// Each of the first `world` threads of the calling block signals one peer and waits for that
// peer's signal. `epoch` must increase by one per use of a channel. Returns false on timeout.
AXB_DEVICE bool peer_barrier_block(const PeerPtrs& pads, int rank, int world, int channel,
                                   unsigned int epoch, int* status,
                                   unsigned long long budget_ns) {
  bool ok = true;
  if ((int)threadIdx.x < world) {
    const int peer = threadIdx.x;
    unsigned int* remote =
        reinterpret_cast<unsigned int*>(pads.p[peer]) + PAD_BASE_WORD + channel * MAX_WORLD + rank;
    __threadfence_system();
    st_release_sys(remote, epoch);
    const unsigned int* mine =
        reinterpret_cast<const unsigned int*>(pads.p[rank]) + PAD_BASE_WORD + channel * MAX_WORLD + peer;
    const uint64_t t0 = global_timer_ns();
    uint32_t spins = 0;
    while ((int)(ld_acquire_sys(mine) - epoch) < 0) {
      if ((++spins & 0x3F) == 0 && global_timer_ns() - t0 > budget_ns) {
        if (status) atomicCAS(status, 0, AXB_TIMEOUT_PEER_FLAG);
        ok = false;
        break;
      }
      __nanosleep(100);
    }
  }
  __syncthreads();
  return ok;
}

__global__ void peer_barrier_kernel(PeerPtrs pads, int rank, int world, int channel,
                                    unsigned int epoch, int* status,
                                    unsigned long long budget_ns) {
  peer_barrier_block(pads, rank, world, channel, epoch, status, budget_ns);
}

AXB_DEVICE float4 multimem_ld_reduce_f32x4(const float* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
AXB_DEVICE void multimem_st_f32x4(float* mc_addr, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr),
               "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}
AXB_DEVICE void multimem_st_b32x2(void* mc_addr, uint32_t a, uint32_t b) {
  asm volatile("multimem.st.relaxed.sys.global.v2.bf16x2 [%0], {%1, %2};" ::"l"(mc_addr), "r"(a),
               "r"(b)
               : "memory");
}

struct RsAdamwParams {
  PeerPtrs grad;     // fp32 [n] symmetric, each rank's local gradient sum
  PeerPtrs master;   // fp32 [n] symmetric
  PeerPtrs shadow;   // bf16 [n] symmetric
  PeerPtrs pads;     // signal pads
  PeerPtrs scratch;  // fp32 [MAX_WORLD] symmetric: per-rank partial squared norms
  float* grad_mc;    // multicast addresses (nullptr -> plain peer loads / stores)
  float* master_mc;
  __nv_bfloat16* shadow_mc;
  float* exp_avg;     // local, full length; only the owned slice is touched
  float* exp_avg_sq;
  long long n;        // multiple of 4 * world
  int rank, world;
  unsigned int epoch;  // barrier epoch base (3 barriers are used: epoch, epoch+1, epoch+2)
  float lr, beta1, beta2, eps, wd, bc1, bc2, max_norm, grad_scale;
  float* gnorm_sq_out;  // local scalar: squared norm of the reduced (unscaled) gradient
  int* status;
  unsigned long long budget_ns;
  // 0: everything in one launch (one parameter group). An optimizer with several groups clips by the
  // norm over ALL of them, so it runs two passes: mode 1 for every group (reduce-scatter, add the
  // group's squared norm to *gnorm_sq_out, leave the reduced slice in place), then mode 2 for every
  // group (clip by *gnorm_sq_out, AdamW, publish; no reduction).
  int mode;
  // 1: the fp32 master exists only on the rank that owns the slice (n / world floats, master.p[rank] is
  // rebased so that the global element index addresses it); only the bf16 copy is published to all ranks
  int master_local;
};

__global__ void __launch_bounds__(256)
    rs_adamw_ag_kernel(const RsAdamwParams p) {
  cg::grid_group grid = cg::this_grid();
  __shared__ float sh[32];
  const long long slice = p.n / p.world;
  const long long lo = slice * p.rank;
  float* my_grad = reinterpret_cast<float*>(p.grad.p[p.rank]);
  const long long nvec = slice / 4;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;

  float total = 0.f;
  if (p.mode != 2) {
  // ---- barrier 1: every rank has finished writing its local gradient
  if (blockIdx.x == 0) peer_barrier_block(p.pads, p.rank, p.world, 0, p.epoch, p.status, p.budget_ns);
  grid.sync();

  // ---- phase B: reduce my slice over all ranks, keep it in my own gradient buffer
  float ss = 0.f;
  if (p.grad_mc) {
    // four independent in-switch reductions in flight per thread (the NVSwitch round trip is the cost)
    constexpr int U = 4;
    for (long long v0 = tid; v0 < nvec; v0 += nthreads * U) {
      float4 g[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long v = v0 + u * nthreads;
        g[u] = multimem_ld_reduce_f32x4(p.grad_mc + lo + (v < nvec ? v : v0) * 4);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long v = v0 + u * nthreads;
        if (v >= nvec) continue;
        *reinterpret_cast<float4*>(my_grad + lo + v * 4) = g[u];
        ss += g[u].x * g[u].x + g[u].y * g[u].y + g[u].z * g[u].z + g[u].w * g[u].w;
      }
    }
  } else {
    for (long long v = tid; v < nvec; v += nthreads) {
      const long long i = lo + v * 4;
      float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < p.world; ++r) {
        const float4 x = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.grad.p[r]) + i);
        g.x += x.x; g.y += x.y; g.z += x.z; g.w += x.w;
      }
      *reinterpret_cast<float4*>(my_grad + i) = g;
      ss += g.x * g.x + g.y * g.y + g.z * g.z + g.w * g.w;
    }
  }
  // block reduce -> atomic into this rank's scratch slot
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float r = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    if (threadIdx.x == 0) atomicAdd(reinterpret_cast<float*>(p.scratch.p[p.rank]) + MAX_WORLD + 0, r);
  }
  grid.sync();
  // ---- publish my partial to every rank's slot [rank], barrier 2
  if (blockIdx.x == 0) {
    if ((int)threadIdx.x < p.world) {
      const float part = *(reinterpret_cast<volatile float*>(p.scratch.p[p.rank]) + MAX_WORLD);
      reinterpret_cast<float*>(p.scratch.p[threadIdx.x])[p.rank] = part;
    }
    __syncthreads();
    peer_barrier_block(p.pads, p.rank, p.world, 0, p.epoch + 1, p.status, p.budget_ns);
  }
  grid.sync();

  {
    const volatile float* parts = reinterpret_cast<const volatile float*>(p.scratch.p[p.rank]);
    for (int r = 0; r < p.world; ++r) total += parts[r];
  }
  if (p.mode == 1) {
    // first pass of a multi-group step: accumulate the norm, clear what the peers have read, stop
    const long long n4 = p.n / 4;
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    const long long s0 = lo / 4, s1 = (lo + slice) / 4;
    for (long long v = tid; v < n4; v += nthreads)
      if (v < s0 || v >= s1) reinterpret_cast<float4*>(my_grad)[v] = z;
    grid.sync();   // every thread has read the partial sums before they are re-armed
    if (tid == 0) {
      if (p.gnorm_sq_out) *p.gnorm_sq_out += total;
      reinterpret_cast<float*>(p.scratch.p[p.rank])[MAX_WORLD] = 0.f;
    }
    return;
  }
  if (tid == 0 && p.gnorm_sq_out) *p.gnorm_sq_out = total;
  } else {
    total = *reinterpret_cast<const volatile float*>(p.gnorm_sq_out);
  }
  // ---- phase C: clip + AdamW on my slice, publish master + shadow to all ranks
  float clip = p.grad_scale;
  if (p.max_norm > 0.f) clip *= fminf(1.f, p.max_norm / (sqrtf(total) * p.grad_scale + 1e-6f));
  float* my_master = reinterpret_cast<float*>(p.master.p[p.rank]);
  for (long long v = tid; v < nvec; v += nthreads) {
    const long long i = lo + v * 4;
    const float4 g4 = *reinterpret_cast<const float4*>(my_grad + i);
    *reinterpret_cast<float4*>(my_grad + i) = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 w4 = *reinterpret_cast<const float4*>(my_master + i);
    float4 m4 = *reinterpret_cast<const float4*>(p.exp_avg + i);
    float4 v4 = *reinterpret_cast<const float4*>(p.exp_avg_sq + i);
    float g[4] = {g4.x * clip, g4.y * clip, g4.z * clip, g4.w * clip};
    float w[4] = {w4.x, w4.y, w4.z, w4.w};
    float m[4] = {m4.x, m4.y, m4.z, m4.w};
    float s[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      m[k] = p.beta1 * m[k] + (1.f - p.beta1) * g[k];
      s[k] = p.beta2 * s[k] + (1.f - p.beta2) * g[k] * g[k];
      w[k] *= (1.f - p.lr * p.wd);
      w[k] -= p.lr * (m[k] / p.bc1) / (sqrtf(s[k] / p.bc2) + p.eps);
    }
    *reinterpret_cast<float4*>(p.exp_avg + i) = make_float4(m[0], m[1], m[2], m[3]);
    *reinterpret_cast<float4*>(p.exp_avg_sq + i) = make_float4(s[0], s[1], s[2], s[3]);
    const float4 wn = make_float4(w[0], w[1], w[2], w[3]);
    const uint32_t b0 = pack_bf16x2(w[0], w[1]), b1 = pack_bf16x2(w[2], w[3]);
    if (p.master_local) {
      *reinterpret_cast<float4*>(my_master + i) = wn;
      if (p.shadow_mc) {
        multimem_st_b32x2(p.shadow_mc + i, b0, b1);
      } else {
        for (int r = 0; r < p.world; ++r)
          *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.shadow.p[r]) + i) = make_uint2(b0, b1);
      }
    } else if (p.master_mc) {
      multimem_st_f32x4(p.master_mc + i, wn);
      multimem_st_b32x2(p.shadow_mc + i, b0, b1);
    } else {
      for (int r = 0; r < p.world; ++r) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.master.p[r]) + i) = wn;
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.shadow.p[r]) + i) = make_uint2(b0, b1);
      }
    }
  }
  // ---- zero the rest of my gradient buffer (peers finished reading it at barrier 2)
  {
    const long long n4 = p.n / 4;
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    const long long s0 = lo / 4, s1 = (lo + slice) / 4;  // my slice is cleared in the loop above
    for (long long v = tid; v < n4; v += nthreads)
      if (v < s0 || v >= s1) reinterpret_cast<float4*>(my_grad)[v] = z;
    if (tid == 0) reinterpret_cast<float*>(p.scratch.p[p.rank])[MAX_WORLD] = 0.f;
  }
  __threadfence_system();
  grid.sync();
  // ---- barrier 3: every rank's parameters are visible everywhere
  if (blockIdx.x == 0)
    peer_barrier_block(p.pads, p.rank, p.world, 0, p.epoch + 2, p.status, p.budget_ns);
}

struct AllreduceParams {
  PeerPtrs buf;  // fp32 [world][n] symmetric staging: slot [src] of every rank
  PeerPtrs pads;
  float* inout;
  int n, rank, world, channel;
  unsigned int epoch;
  int* status;
  unsigned long long budget_ns;
};

// one-shot all-reduce for small vectors (n <= 1024): write my vector into slot [rank] of every
// peer, barrier, sum the slots locally.
__global__ void peer_allreduce_kernel(const AllreduceParams p) {
  for (int r = 0; r < p.world; ++r) {
    float* dst = reinterpret_cast<float*>(p.buf.p[r]) + (long long)p.rank * p.n;
    for (int i = threadIdx.x; i < p.n; i += blockDim.x) dst[i] = p.inout[i];
  }
  __syncthreads();
  peer_barrier_block(p.pads, p.rank, p.world, p.channel, p.epoch, p.status, p.budget_ns);
  const volatile float* mine = reinterpret_cast<const volatile float*>(p.buf.p[p.rank]);
  for (int i = threadIdx.x; i < p.n; i += blockDim.x) {
    float s = 0.f;
    for (int r = 0; r < p.world; ++r) s += mine[(long long)r * p.n + i];
    p.inout[i] = s;
  }
  __syncthreads();
  // second barrier so a later call cannot overwrite slots that are still being read
  peer_barrier_block(p.pads, p.rank, p.world, p.channel, p.epoch + 1, p.status, p.budget_ns);
}

int fill_ptrs(PeerPtrs& dst, const unsigned long long* src, int world) {
  if (world > MAX_WORLD || world < 1) return -2;
  for (int i = 0; i < MAX_WORLD; ++i) dst.p[i] = i < world ? src[i] : 0ull;
  return 0;
}

}  // namespace

extern "C" int axb_peer_barrier(const unsigned long long* pad_ptrs, int rank, int world,
                                int channel, unsigned int epoch, int* status, long long budget_ns,
                                void* stream) {
  PeerPtrs pads;
  if (fill_ptrs(pads, pad_ptrs, world)) return -2;
  peer_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      pads, rank, world, channel, epoch, status, (unsigned long long)budget_ns);
  return (int)cudaGetLastError();
}

// All *_ptrs arguments are HOST arrays of `world` peer-mapped device addresses.
static int rs_adamw_ag_impl(const unsigned long long* grad_ptrs,
                               const unsigned long long* master_ptrs,
                               const unsigned long long* shadow_ptrs,
                               const unsigned long long* pad_ptrs,
                               const unsigned long long* scratch_ptrs, void* grad_mc,
                               void* master_mc, void* shadow_mc, float* exp_avg, float* exp_avg_sq,
                               long long n, int rank, int world, unsigned int epoch, float lr,
                               float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                               float max_norm, float grad_scale, float* gnorm_sq_out, int* status,
                               long long budget_ns, void* stream, int sliced_moments, int mode = 0) {
  if (n % (4LL * world)) return -3;
  if (mode < 0 || mode > 2 || (mode != 0 && gnorm_sq_out == nullptr)) return -2;
  RsAdamwParams p;
  p.mode = mode;
  if (fill_ptrs(p.grad, grad_ptrs, world) || fill_ptrs(p.master, master_ptrs, world) ||
      fill_ptrs(p.shadow, shadow_ptrs, world) || fill_ptrs(p.pads, pad_ptrs, world) ||
      fill_ptrs(p.scratch, scratch_ptrs, world))
    return -2;
  p.master_local = (sliced_moments & 2) ? 1 : 0;
  p.grad_mc = reinterpret_cast<float*>(grad_mc);
  p.master_mc = reinterpret_cast<float*>(master_mc);
  p.shadow_mc = reinterpret_cast<__nv_bfloat16*>(shadow_mc);
  if (!(p.grad_mc && (p.master_mc || p.master_local) && p.shadow_mc)) {
    p.grad_mc = nullptr;
    p.master_mc = nullptr;
    p.shadow_mc = nullptr;
  }
  if (p.master_local) {
    // master_ptrs[rank] is this rank's [n / world] slice: rebase it to the global element index
    p.master_mc = nullptr;
    p.master.p[rank] -= (unsigned long long)((n / world) * (long long)rank) * sizeof(float);
  }
  // ZeRO-style moments: each rank stores only the n / world elements it updates; the kernel
  // indexes moments with the global element index, so rebase the pointers by the slice start.
  const long long slice_lo = (sliced_moments & 1) ? (n / world) * (long long)rank : 0;
  p.exp_avg = exp_avg - slice_lo;
  p.exp_avg_sq = exp_avg_sq - slice_lo;
  p.n = n;
  p.rank = rank;
  p.world = world;
  p.epoch = epoch;
  p.lr = lr; p.beta1 = beta1; p.beta2 = beta2; p.eps = eps; p.wd = wd; p.bc1 = bc1; p.bc2 = bc2;
  p.max_norm = max_norm;
  p.grad_scale = grad_scale;
  p.gnorm_sq_out = gnorm_sq_out;
  p.status = status;
  p.budget_ns = (unsigned long long)budget_ns;
  int dev = 0, sms = 0, per_sm = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, rs_adamw_ag_kernel, 256, 0);
  if (per_sm < 1) return -4;
  int grid = sms * (per_sm > 2 ? 2 : per_sm);
  void* args[] = {(void*)&p};
  cudaError_t e = cudaLaunchCooperativeKernel((void*)rs_adamw_ag_kernel, dim3(grid), dim3(256), args,
                                              0, reinterpret_cast<cudaStream_t>(stream));
  return (int)e;
}

// exp_avg / exp_avg_sq: full-length local arrays (only the owned slice is touched)
extern "C" int axb_rs_adamw_ag(const unsigned long long* grad_ptrs, const unsigned long long* master_ptrs,
                               const unsigned long long* shadow_ptrs, const unsigned long long* pad_ptrs,
                               const unsigned long long* scratch_ptrs, void* grad_mc, void* master_mc,
                               void* shadow_mc, float* exp_avg, float* exp_avg_sq, long long n, int rank, int world,
                               unsigned int epoch, float lr, float beta1, float beta2, float eps, float wd, float bc1,
                               float bc2, float max_norm, float grad_scale, float* gnorm_sq_out, int* status,
                               long long budget_ns, void* stream) {
  return rs_adamw_ag_impl(grad_ptrs, master_ptrs, shadow_ptrs, pad_ptrs, scratch_ptrs, grad_mc, master_mc, shadow_mc,
                          exp_avg, exp_avg_sq, n, rank, world, epoch, lr, beta1, beta2, eps, wd, bc1, bc2, max_norm,
                          grad_scale, gnorm_sq_out, status, budget_ns, stream, 0);
}

// Same, with exp_avg / exp_avg_sq holding only this rank's slice (n / world elements each).
extern "C" int axb_rs_adamw_ag_sharded(const unsigned long long* grad_ptrs, const unsigned long long* master_ptrs,
                                       const unsigned long long* shadow_ptrs, const unsigned long long* pad_ptrs,
                                       const unsigned long long* scratch_ptrs, void* grad_mc, void* master_mc,
                                       void* shadow_mc, float* exp_avg, float* exp_avg_sq, long long n, int rank,
                                       int world, unsigned int epoch, float lr, float beta1, float beta2, float eps,
                                       float wd, float bc1, float bc2, float max_norm, float grad_scale,
                                       float* gnorm_sq_out, int* status, long long budget_ns, void* stream) {
  return rs_adamw_ag_impl(grad_ptrs, master_ptrs, shadow_ptrs, pad_ptrs, scratch_ptrs, grad_mc, master_mc, shadow_mc,
                          exp_avg, exp_avg_sq, n, rank, world, epoch, lr, beta1, beta2, eps, wd, bc1, bc2, max_norm,
                          grad_scale, gnorm_sq_out, status, budget_ns, stream, 1);
}

// Two-pass form for optimizers with several parameter groups (see RsAdamwParams::mode): call with
// mode 1 for every group after zeroing *gnorm_sq_out, then with mode 2 for every group. Each call
// consumes three barrier epochs like the one-launch form. sliced_moments: bit 0 = exp_avg / exp_avg_sq hold
// only this rank's slice; bit 1 = the fp32 master does too (master_ptrs[rank] points at that slice, the
// other entries are ignored) and only the bf16 copy is published.
extern "C" int axb_rs_adamw_ag_pass(const unsigned long long* grad_ptrs, const unsigned long long* master_ptrs,
                                    const unsigned long long* shadow_ptrs, const unsigned long long* pad_ptrs,
                                    const unsigned long long* scratch_ptrs, void* grad_mc, void* master_mc,
                                    void* shadow_mc, float* exp_avg, float* exp_avg_sq, long long n, int rank,
                                    int world, unsigned int epoch, float lr, float beta1, float beta2, float eps,
                                    float wd, float bc1, float bc2, float max_norm, float grad_scale,
                                    float* gnorm_sq_out, int* status, long long budget_ns, void* stream,
                                    int sliced_moments, int mode) {
  return rs_adamw_ag_impl(grad_ptrs, master_ptrs, shadow_ptrs, pad_ptrs, scratch_ptrs, grad_mc, master_mc, shadow_mc,
                          exp_avg, exp_avg_sq, n, rank, world, epoch, lr, beta1, beta2, eps, wd, bc1, bc2, max_norm,
                          grad_scale, gnorm_sq_out, status, budget_ns, stream, sliced_moments, mode);
}

extern "C" int axb_peer_allreduce_f32(const unsigned long long* buf_ptrs,
                                      const unsigned long long* pad_ptrs, float* inout, int n,
                                      int rank, int world, int channel, unsigned int epoch,
                                      int* status, long long budget_ns, void* stream) {
  if (n > 1024) return -3;
  AllreduceParams p;
  if (fill_ptrs(p.buf, buf_ptrs, world) || fill_ptrs(p.pads, pad_ptrs, world)) return -2;
  p.inout = inout;
  p.n = n;
  p.rank = rank;
  p.world = world;
  p.channel = channel;
  p.epoch = epoch;
  p.status = status;
  p.budget_ns = (unsigned long long)budget_ns;
  peer_allreduce_kernel<<<1, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// All-gather by store: every rank writes its [rows, width] bf16 block (row stride src_ld) into
// rows [row_off, row_off + rows) of the symmetric [*, width] buffer of EVERY rank, through the
// NVSwitch multicast address (multimem.st) or plain peer stores. Used to publish the rotated K / V
// rows of a context-parallel rank to all ranks before attention.
namespace {
__global__ void allgather_store_kernel(const __nv_bfloat16* __restrict__ src, long long src_ld, long long rows,
                                       int width, long long row_off, __nv_bfloat16* mc, PeerPtrs dst, int world) {
  const int vec_per_row = width / 8;
  const long long n = rows * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = (int)(i % vec_per_row) * 8;
    const uint4 v = *reinterpret_cast<const uint4*>(src + r * src_ld + c);
    const long long off = (row_off + r) * width + c;
    if (mc) {
      asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc + off), "r"(v.x),
                   "r"(v.y), "r"(v.z), "r"(v.w)
                   : "memory");
    } else {
      for (int p = 0; p < world; ++p) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dst.p[p]) + off) = v;
    }
  }
}
}  // namespace

extern "C" int axb_allgather_store(const void* src, long long src_ld, long long rows, int width, long long row_off,
                                   void* mc, const unsigned long long* dst_ptrs, int world, void* stream) {
  if (rows <= 0) return 0;
  if ((width & 7) || (src_ld & 7)) return -2;
  PeerPtrs dst;
  if (fill_ptrs(dst, dst_ptrs, world)) return -2;
  const long long n = rows * (width / 8);
  int grid = (int)((n + 255) / 256 > 148 * 8 ? 148 * 8 : (n + 255) / 256);
  allgather_store_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const __nv_bfloat16*)src, src_ld, rows, width, row_off, (__nv_bfloat16*)mc, dst, world);
  return (int)cudaGetLastError();
}
