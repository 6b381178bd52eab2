// Peer-memory collectives over NVLink / NVSwitch for the data-parallel path, written as plain
// sm_100a kernels on symmetric buffers (every rank maps every peer's buffer at the same offsets):
//
//   * bucket reduce-scatter fused with the 1/W (x loss scale) multiply and the squared-norm
//     partial of the reduced shard: each rank sums ITS shard of the bucket over all peers,
//     either with one in-switch reduction per 16 bytes (multimem.ld_reduce on the NVLS multicast
//     mapping) or with W plain peer loads, and writes the result in place into its own buffer;
//   * bucket all-gather of updated bf16 parameters: each rank pushes its shard into every
//     peer's parameter buffer (multimem.st, or W plain peer stores);
//   * a flag barrier between ranks: a rank signals by storing a monotonically increasing epoch
//     into a slot of every peer's flag array (st.release.sys) and waits for its own slots
//     (ld.acquire.sys). Every wait is bounded by a time limit passed by the host; a wait that
//     runs out records FT_ERR_WAIT_PEER in the status word, and the kernel still terminates.
//
// Stand in for the reference's NCCL reduce_scatter_tensor / all_gather_into_tensor / all_reduce
// calls plus the aten scale, cast and norm kernels around them
// (exports/train_engine_0.5B/src/training_engine_tensor/nccl.py:1093-1137, 1357-1390, 1454-1513).
#include "ptx.cuh"

namespace ft {

constexpr int COMM_MAX_RANKS = 16;
constexpr int COMM_THREADS = 512;

struct CommPeers {
  void* buf[COMM_MAX_RANKS];         // peer base pointers of the data buffer
  uint32_t* flags[COMM_MAX_RANKS];   // peer base pointers of the flag arrays [slots][world]
  void* mc;                          // multicast mapping of the data buffer (nullptr: none)
  // Per-slot epoch base in device memory (nullptr: none). The epoch a kernel signals / waits for
  // is its launch argument plus this base, so a captured CUDA graph can be replayed: its
  // launch arguments stay fixed while a kernel at the end of the graph advances the base.
  const uint32_t* ebase;
  int rank, world;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const void* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_b32x4(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}
__device__ __forceinline__ float4 ld_peer_f32x4(const float* p) {
  float4 v;
  asm volatile("ld.global.relaxed.sys.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_peer_b32x4(void* p, uint4 v) {
  asm volatile("st.global.relaxed.sys.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// Signal `epoch` into slot [slot][rank] of every peer (threads 0..world-1 of the calling CTA).
__device__ __forceinline__ void signal_peers(const CommPeers& c, int slot, uint32_t epoch) {
  if (threadIdx.x < c.world) {
    if (c.ebase) epoch += c.ebase[slot];
    __threadfence_system();
    st_release_sys(c.flags[threadIdx.x] + slot * c.world + c.rank, epoch);
  }
}

// Wait until every peer has signalled at least `epoch` into this rank's slot. Bounded:
// returns false (and records the status) when `limit_ns` passes first. Whole CTA must call.
__device__ __forceinline__ bool wait_peers(const CommPeers& c, int slot, uint32_t epoch,
                                           uint64_t limit_ns, int* status) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  if (threadIdx.x < c.world) {
    if (c.ebase) epoch += c.ebase[slot];
    const uint32_t* f = c.flags[c.rank] + slot * c.world + threadIdx.x;
    const uint64_t t0 = globaltimer_ns();
    while (true) {
      // epochs only grow; the signed difference is safe across 32-bit wrap-around
      if (static_cast<int32_t>(ld_acquire_sys(f) - epoch) >= 0) break;
      if (globaltimer_ns() - t0 > limit_ns) {
        s_fail = 1;
        if (status) atomicCAS(status, 0, FT_ERR_WAIT_PEER);
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  return s_fail == 0;
}

// ---------------------------------------------------------------------------------------
// Barrier only (used by tests of the timeout path and as a building block).
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(COMM_THREADS)
peer_barrier_kernel(CommPeers c, int slot, uint32_t epoch, uint64_t limit_ns, int do_signal,
                    int* status) {
  if (do_signal) signal_peers(c, slot, epoch);
  wait_peers(c, slot, epoch, limit_ns, status);
}

// ---------------------------------------------------------------------------------------
// Reduce-scatter of one bucket, in place, fused with scale and squared-norm partial.
//   bucket = elements [start, start + n_per_rank * world) of the fp32 buffer; this rank owns
//   [start + rank*n_per_rank, +n_per_rank). n_per_rank % 4 == 0.
// Protocol: entry barrier (slot 0) -> reduce -> exit barrier (slot 1, last CTA to finish).
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(COMM_THREADS)
bucket_reduce_scatter_kernel(CommPeers c, long start, long n_per_rank, float scale,
                             float* __restrict__ sumsq, uint32_t epoch, uint64_t limit_ns,
                             unsigned int* __restrict__ done_ctr, int* status) {
  __shared__ float red[COMM_THREADS / 32];
  if (blockIdx.x == 0) signal_peers(c, 0, epoch);
  const bool ok = wait_peers(c, 0, epoch, limit_ns, status);
  float ss = 0.f;
  if (ok) {
    const long base = start + static_cast<long>(c.rank) * n_per_rank;
    float* mine = static_cast<float*>(c.buf[c.rank]) + base;
    const long nvec = n_per_rank / 4;
    constexpr int U = 4;  // independent 16-byte requests in flight per thread
    const long stride = static_cast<long>(gridDim.x) * COMM_THREADS;
    const long i0 = static_cast<long>(blockIdx.x) * COMM_THREADS + threadIdx.x;
    if (c.mc) {
      const float* mc = static_cast<const float*>(c.mc) + base;
      for (long i = i0; i < nvec; i += stride * U) {
        float4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (i + u * stride < nvec) v[u] = multimem_ld_reduce_f32x4(mc + 4 * (i + u * stride));
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (i + u * stride < nvec) {
            float4 w = v[u];
            w.x *= scale; w.y *= scale; w.z *= scale; w.w *= scale;
            ss += w.x * w.x + w.y * w.y + w.z * w.z + w.w * w.w;
            reinterpret_cast<float4*>(mine)[i + u * stride] = w;
          }
      }
    } else {
      for (long i = i0; i < nvec; i += stride * U) {
        float4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int p = 0; p < c.world; ++p) {
          const int q = (c.rank + p) % c.world;  // start at self, spread the peers
          const float* src = static_cast<const float*>(c.buf[q]) + base;
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (i + u * stride < nvec) {
              const float4 a = ld_peer_f32x4(src + 4 * (i + u * stride));
              v[u].x += a.x; v[u].y += a.y; v[u].z += a.z; v[u].w += a.w;
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (i + u * stride < nvec) {
            float4 w = v[u];
            w.x *= scale; w.y *= scale; w.z *= scale; w.w *= scale;
            ss += w.x * w.x + w.y * w.y + w.z * w.z + w.w * w.w;
            reinterpret_cast<float4*>(mine)[i + u * stride] = w;
          }
      }
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < COMM_THREADS / 32 ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0 && sumsq) atomicAdd(sumsq, t);
  }
  // exit barrier: the last CTA of this rank tells the peers that it no longer reads their
  // memory and waits until no peer reads ours, so later kernels may overwrite the bucket.
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int prev = atomicAdd(done_ctr, 1u);
    s_last = (prev == gridDim.x - 1) ? 1 : 0;
    if (s_last) *done_ctr = 0;  // re-arm for the next launch (stream-ordered)
  }
  __syncthreads();
  if (s_last) {
    signal_peers(c, 1, epoch);
    wait_peers(c, 1, epoch, limit_ns, status);
  }
}

// ---------------------------------------------------------------------------------------
// All-gather of one bucket of 2-byte parameters: push this rank's shard to every peer.
//   shard = elements [start + rank*n_per_rank, +n_per_rank) of the bf16 buffer (already holds
//   the new values locally). n_per_rank % 8 == 0. Exit barrier on slot 2.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(COMM_THREADS)
bucket_all_gather_kernel(CommPeers c, long start, long n_per_rank, uint32_t epoch,
                         uint64_t limit_ns, unsigned int* __restrict__ done_ctr, int* status) {
  const long base = start + static_cast<long>(c.rank) * n_per_rank;  // in 2-byte elements
  const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(c.buf[c.rank]) + base);
  const long nvec = n_per_rank / 8;
  constexpr int U = 4;
  const long stride = static_cast<long>(gridDim.x) * COMM_THREADS;
  const long i0 = static_cast<long>(blockIdx.x) * COMM_THREADS + threadIdx.x;
  if (c.mc) {
    uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(c.mc) + base);
    for (long i = i0; i < nvec; i += stride * U) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i + u * stride < nvec) v[u] = src[i + u * stride];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i + u * stride < nvec) multimem_st_b32x4(dst + i + u * stride, v[u]);
    }
  } else {
    for (long i = i0; i < nvec; i += stride * U) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i + u * stride < nvec) v[u] = src[i + u * stride];
      for (int p = 1; p < c.world; ++p) {
        const int q = (c.rank + p) % c.world;
        uint4* dq = reinterpret_cast<uint4*>(static_cast<uint16_t*>(c.buf[q]) + base);
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (i + u * stride < nvec) st_peer_b32x4(dq + i + u * stride, v[u]);
      }
    }
  }
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int prev = atomicAdd(done_ctr, 1u);
    s_last = (prev == gridDim.x - 1) ? 1 : 0;
    if (s_last) *done_ctr = 0;
  }
  __syncthreads();
  if (s_last) {
    signal_peers(c, 2, epoch);
    wait_peers(c, 2, epoch, limit_ns, status);
  }
}

// ---------------------------------------------------------------------------------------
// AdamW shard update fused with the parameter all-gather: every thread updates eight master
// weights (fp32 p / m / v, decoupled weight decay, bias correction, clip from hyper[6]) and
// stores the eight bf16 results straight into EVERY rank's parameter buffer, by one
// `multimem.st` through the switch or by one 16-byte store per peer, so the updated shard is
// never re-read for a separate gather. Exit barrier on slot 2 as in the plain all-gather.
//   shard = elements [start + rank*n_per_rank, +n_per_rank); n_per_rank % 8 == 0.
//   hyper = {lr, beta1, beta2, eps, bias_corr1, bias_corr2, clip, _} in device memory;
//   seg_end[s] = exclusive end offset of segment s within the shard, seg_wd, seg_lr_mult.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(COMM_THREADS)
adamw_all_gather_kernel(CommPeers c, long start, long n_per_rank, float* __restrict__ p32,
                        float* __restrict__ m, float* __restrict__ v,
                        const float* __restrict__ g, const float* __restrict__ hyper,
                        const long* __restrict__ seg_end, const float* __restrict__ seg_wd,
                        const float* __restrict__ seg_lr_mult, int nseg, uint32_t epoch,
                        uint64_t limit_ns, unsigned int* __restrict__ done_ctr, int* status) {
  const float lr = hyper[0], b1 = hyper[1], b2 = hyper[2], eps = hyper[3];
  const float inv_bc1 = 1.f / hyper[4], inv_bc2 = 1.f / hyper[5], clip = hyper[6];
  const long base = start + static_cast<long>(c.rank) * n_per_rank;  // in elements
  const long nvec = n_per_rank / 8;
  for (long i = static_cast<long>(blockIdx.x) * COMM_THREADS + threadIdx.x; i < nvec;
       i += static_cast<long>(gridDim.x) * COMM_THREADS) {
    const long e0 = i * 8;
    int lo = 0, hi = nseg - 1;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (seg_end[mid] > e0) hi = mid; else lo = mid + 1;
    }
    int seg = lo;
    float pp[8], mm[8], vv[8], gg[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float4 a = reinterpret_cast<const float4*>(p32)[2 * i + h];
      const float4 b = reinterpret_cast<const float4*>(m)[2 * i + h];
      const float4 d = reinterpret_cast<const float4*>(v)[2 * i + h];
      const float4 e = reinterpret_cast<const float4*>(g)[2 * i + h];
      pp[4 * h] = a.x; pp[4 * h + 1] = a.y; pp[4 * h + 2] = a.z; pp[4 * h + 3] = a.w;
      mm[4 * h] = b.x; mm[4 * h + 1] = b.y; mm[4 * h + 2] = b.z; mm[4 * h + 3] = b.w;
      vv[4 * h] = d.x; vv[4 * h + 1] = d.y; vv[4 * h + 2] = d.z; vv[4 * h + 3] = d.w;
      gg[4 * h] = e.x; gg[4 * h + 1] = e.y; gg[4 * h + 2] = e.z; gg[4 * h + 3] = e.w;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      while (seg < nseg - 1 && seg_end[seg] <= e0 + k) ++seg;
      const float wd = seg_wd[seg], lrm = seg_lr_mult[seg];
      const float gr = gg[k] * clip;
      mm[k] = b1 * mm[k] + (1.f - b1) * gr;
      vv[k] = b2 * vv[k] + (1.f - b2) * gr * gr;
      const float upd = (mm[k] * inv_bc1) / (sqrtf(vv[k] * inv_bc2) + eps) + wd * pp[k];
      pp[k] -= lr * lrm * upd;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      reinterpret_cast<float4*>(p32)[2 * i + h] =
          make_float4(pp[4 * h], pp[4 * h + 1], pp[4 * h + 2], pp[4 * h + 3]);
      reinterpret_cast<float4*>(m)[2 * i + h] =
          make_float4(mm[4 * h], mm[4 * h + 1], mm[4 * h + 2], mm[4 * h + 3]);
      reinterpret_cast<float4*>(v)[2 * i + h] =
          make_float4(vv[4 * h], vv[4 * h + 1], vv[4 * h + 2], vv[4 * h + 3]);
    }
    uint4 o;
    o.x = pack2_bf16(pp[0], pp[1]);
    o.y = pack2_bf16(pp[2], pp[3]);
    o.z = pack2_bf16(pp[4], pp[5]);
    o.w = pack2_bf16(pp[6], pp[7]);
    if (c.mc) {
      multimem_st_b32x4(reinterpret_cast<uint4*>(static_cast<uint16_t*>(c.mc) + base) + i, o);
    } else {
      for (int p = 0; p < c.world; ++p) {
        const int q = (c.rank + p) % c.world;
        st_peer_b32x4(reinterpret_cast<uint4*>(static_cast<uint16_t*>(c.buf[q]) + base) + i, o);
      }
    }
  }
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int prev = atomicAdd(done_ctr, 1u);
    s_last = (prev == gridDim.x - 1) ? 1 : 0;
    if (s_last) *done_ctr = 0;
  }
  __syncthreads();
  if (s_last) {
    signal_peers(c, 2, epoch);
    wait_peers(c, 2, epoch, limit_ns, status);
  }
}

// ---------------------------------------------------------------------------------------
// Small all-reduce (sum) of a few floats through the flag-protected symmetric scratch area:
// every rank writes its values into its own slot of every peer, barrier, each rank sums.
//   scratch layout per rank: [world][n] floats at float offset `scratch_off`. n <= 64.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(COMM_THREADS)
small_all_reduce_kernel(CommPeers c, long scratch_off, float* __restrict__ vals, int n,
                        uint32_t epoch, uint64_t limit_ns, int* status) {
  const int tid = threadIdx.x;
  for (int i = tid; i < n * c.world; i += COMM_THREADS) {
    const int p = i / n, k = i % n;
    float* dst = static_cast<float*>(c.buf[p]) + scratch_off + static_cast<long>(c.rank) * n + k;
    asm volatile("st.global.relaxed.sys.f32 [%0], %1;" ::"l"(dst), "f"(vals[k]) : "memory");
  }
  __syncthreads();
  signal_peers(c, 3, epoch);
  const bool ok = wait_peers(c, 3, epoch, limit_ns, status);
  if (ok && tid < n) {
    const float* mine = static_cast<const float*>(c.buf[c.rank]) + scratch_off;
    float s = 0.f;
    for (int p = 0; p < c.world; ++p) {
      float v;
      asm volatile("ld.global.relaxed.sys.f32 %0, [%1];" : "=f"(v) : "l"(mine + p * n + tid) : "memory");
      s += v;
    }
    vals[tid] = s;
  }
  // second phase so that nobody overwrites a slot that a slower peer has not read yet
  __syncthreads();
  signal_peers(c, 4, epoch);
  wait_peers(c, 4, epoch, limit_ns, status);
}

// ---------------------------------------------------------------------------------------
// Vocab-parallel cross-entropy: exchange of the per-row statistics between tensor-parallel ranks
// inside one kernel. Every rank has written (row max, sum-exp relative to that max, target
// logit or 0) for its vocabulary shard as stats[3][T] at float offset `off` of its symmetric
// buffer. After an entry barrier each rank reads every peer's three vectors with plain peer
// loads and combines them: gmax = max_r m_r, gsum = sum_r s_r * exp(m_r - gmax),
// gtarget = sum_r t_r; writes the combined [3][T] to `combined` (local) and the masked row
// loss log(gsum) + gmax - gtarget to `row_loss`. An exit barrier keeps peers from rewriting
// their statistics before everyone has read them. Replaces the MAX + SUM all-reduce pair of
// exports/train_engine_8b/src/training_engine_tensor/backward.py:203-346.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
ce_stats_exchange_kernel(CommPeers c, long off, int T, const float* __restrict__ mask,
                         float* __restrict__ combined, float* __restrict__ row_loss,
                         uint32_t epoch, uint64_t limit_ns, unsigned int* __restrict__ done_ctr,
                         int* status) {
  if (blockIdx.x == 0) signal_peers(c, 5, epoch);
  const bool ok = wait_peers(c, 5, epoch, limit_ns, status);
  if (ok) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < T; i += gridDim.x * blockDim.x) {
      float m[COMM_MAX_RANKS], sx[COMM_MAX_RANKS];
      float gmax = -INFINITY, gt = 0.f;
      for (int r = 0; r < c.world; ++r) {
        const float* st = static_cast<const float*>(c.buf[r]) + off;
        float t;
        asm volatile("ld.global.relaxed.sys.f32 %0, [%1];" : "=f"(m[r]) : "l"(st + i) : "memory");
        asm volatile("ld.global.relaxed.sys.f32 %0, [%1];" : "=f"(sx[r]) : "l"(st + T + i) : "memory");
        asm volatile("ld.global.relaxed.sys.f32 %0, [%1];" : "=f"(t) : "l"(st + 2 * T + i) : "memory");
        gmax = fmaxf(gmax, m[r]);
        gt += t;
      }
      float gs = 0.f;
      for (int r = 0; r < c.world; ++r) gs += sx[r] * __expf(m[r] - gmax);
      combined[i] = gmax;
      combined[T + i] = gs;
      combined[2 * T + i] = gt;
      if (row_loss) row_loss[i] = (logf(gs) + gmax - gt) * (mask ? mask[i] : 1.f);
    }
  }
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int prev = atomicAdd(done_ctr, 1u);
    s_last = (prev == gridDim.x - 1) ? 1 : 0;
    if (s_last) *done_ctr = 0;
  }
  __syncthreads();
  if (s_last) {
    signal_peers(c, 6, epoch);
    wait_peers(c, 6, epoch, limit_ns, status);
  }
}

// base[slot] += add[slot] for the eight flag slots; the last node of a captured step.
__global__ void epoch_advance_kernel(uint32_t* base, uint32_t a0, uint32_t a1, uint32_t a2,
                                     uint32_t a3, uint32_t a4, uint32_t a5, uint32_t a6,
                                     uint32_t a7) {
  const uint32_t add[8] = {a0, a1, a2, a3, a4, a5, a6, a7};
  if (threadIdx.x < 8) base[threadIdx.x] += add[threadIdx.x];
}

}  // namespace ft

using namespace ft;

#include <mutex>
#include <unordered_map>
// epoch-base registry: this rank's flag array -> device array of 8 per-slot bases
static std::mutex g_ebase_mu;
static std::unordered_map<const void*, const uint32_t*> g_ebase;

// Every later launch whose flag array (own rank's mapping) is `self_flags` adds ebase[slot] to
// its epoch argument. ebase == nullptr removes the entry.
extern "C" int ft_comm_set_epoch_base(const void* self_flags, const void* ebase) {
  std::lock_guard<std::mutex> g(g_ebase_mu);
  if (ebase) g_ebase[self_flags] = static_cast<const uint32_t*>(ebase);
  else g_ebase.erase(self_flags);
  return 0;
}

extern "C" int ft_comm_epoch_advance(void* ebase, const unsigned int* add8, cudaStream_t st) {
  epoch_advance_kernel<<<1, 32, 0, st>>>(static_cast<uint32_t*>(ebase), add8[0], add8[1], add8[2],
                                         add8[3], add8[4], add8[5], add8[6], add8[7]);
  return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

static void fill_peers(CommPeers& c, const void* const* bufs, const void* const* flags, void* mc,
                       int rank, int world) {
  {
    std::lock_guard<std::mutex> g(g_ebase_mu);
    auto it = g_ebase.find(flags[rank]);
    c.ebase = it == g_ebase.end() ? nullptr : it->second;
  }
  for (int i = 0; i < COMM_MAX_RANKS; ++i) {
    c.buf[i] = i < world ? const_cast<void*>(bufs[i]) : nullptr;
    c.flags[i] = i < world ? static_cast<uint32_t*>(const_cast<void*>(flags[i])) : nullptr;
  }
  c.mc = mc;
  c.rank = rank;
  c.world = world;
}

// bufs / flags: host arrays of `world` device pointers (peer mappings, own rank included).
// The flag array of every rank holds at least 8 * world uint32 (zero-initialised once).
extern "C" int ft_peer_barrier(const void* const* flags, int rank, int world, int slot,
                               unsigned int epoch, unsigned long long limit_ns, int do_signal,
                               int* status, cudaStream_t st) {
  if (world > COMM_MAX_RANKS || slot < 0 || slot > 7) return -1;
  CommPeers c;
  fill_peers(c, flags, flags, nullptr, rank, world);
  peer_barrier_kernel<<<1, COMM_THREADS, 0, st>>>(c, slot, epoch, limit_ns, do_signal, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

extern "C" int ft_bucket_reduce_scatter(const void* const* bufs, const void* const* flags, void* mc,
                                        int rank, int world, long start, long n_per_rank,
                                        float scale, void* sumsq, unsigned int epoch,
                                        unsigned long long limit_ns, void* done_ctr, int ctas,
                                        int* status, cudaStream_t st) {
  if (world > COMM_MAX_RANKS || n_per_rank % 4) return -1;
  CommPeers c;
  fill_peers(c, bufs, flags, mc, rank, world);
  if (ctas <= 0) ctas = 96;
  const long need = (n_per_rank / 16 + COMM_THREADS - 1) / COMM_THREADS;
  if (ctas > need) ctas = need < 1 ? 1 : static_cast<int>(need);
  bucket_reduce_scatter_kernel<<<ctas, COMM_THREADS, 0, st>>>(
      c, start, n_per_rank, scale, static_cast<float*>(sumsq), epoch, limit_ns,
      static_cast<unsigned int*>(done_ctr), status);
  return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

extern "C" int ft_bucket_all_gather(const void* const* bufs, const void* const* flags, void* mc,
                                    int rank, int world, long start, long n_per_rank,
                                    unsigned int epoch, unsigned long long limit_ns,
                                    void* done_ctr, int ctas, int* status, cudaStream_t st) {
  if (world > COMM_MAX_RANKS || n_per_rank % 8) return -1;
  CommPeers c;
  fill_peers(c, bufs, flags, mc, rank, world);
  if (ctas <= 0) ctas = 96;
  const long need = (n_per_rank / 32 + COMM_THREADS - 1) / COMM_THREADS;
  if (ctas > need) ctas = need < 1 ? 1 : static_cast<int>(need);
  bucket_all_gather_kernel<<<ctas, COMM_THREADS, 0, st>>>(c, start, n_per_rank, epoch, limit_ns,
                                                          static_cast<unsigned int*>(done_ctr),
                                                          status);
  return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

// Fused AdamW + parameter all-gather of one bucket shard (see adamw_all_gather_kernel).
// bufs: peer mappings of the bf16 parameter buffer; p32 / m / v / g: this rank's fp32 shard.
extern "C" int ft_adamw_all_gather(const void* const* bufs, const void* const* flags, void* mc,
                                   int rank, int world, long start, long n_per_rank, void* p32,
                                   void* m, void* v, const void* g, const void* hyper,
                                   const void* seg_end, const void* seg_wd,
                                   const void* seg_lr_mult, int nseg, unsigned int epoch,
                                   unsigned long long limit_ns, void* done_ctr, int ctas,
                                   int* status, cudaStream_t st) {
  if (world > COMM_MAX_RANKS || n_per_rank % 8 || nseg < 1) return -1;
  CommPeers c;
  fill_peers(c, bufs, flags, mc, rank, world);
  if (ctas <= 0) ctas = 148 * 4;
  const long need = (n_per_rank / 8 + COMM_THREADS - 1) / COMM_THREADS;
  if (ctas > need) ctas = need < 1 ? 1 : static_cast<int>(need);
  adamw_all_gather_kernel<<<ctas, COMM_THREADS, 0, st>>>(
      c, start, n_per_rank, static_cast<float*>(p32), static_cast<float*>(m),
      static_cast<float*>(v), static_cast<const float*>(g), static_cast<const float*>(hyper),
      static_cast<const long*>(seg_end), static_cast<const float*>(seg_wd),
      static_cast<const float*>(seg_lr_mult), nseg, epoch, limit_ns,
      static_cast<unsigned int*>(done_ctr), status);
  return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

extern "C" int ft_small_all_reduce(const void* const* bufs, const void* const* flags, int rank,
                                   int world, long scratch_off, void* vals, int n,
                                   unsigned int epoch, unsigned long long limit_ns, int* status,
                                   cudaStream_t st) {
  if (world > COMM_MAX_RANKS || n > 64 || n < 1) return -1;
  CommPeers c;
  fill_peers(c, bufs, flags, nullptr, rank, world);
  small_all_reduce_kernel<<<1, COMM_THREADS, 0, st>>>(c, scratch_off, static_cast<float*>(vals), n,
                                                      epoch, limit_ns, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

// stats: peer mappings of the symmetric buffer that holds every rank's [3][T] statistics at
// float offset `off`; combined / row_loss: local outputs ([3][T] and [T] floats).
extern "C" int ft_ce_stats_exchange(const void* const* bufs, const void* const* flags, int rank,
                                    int world, long off, int T, const void* mask, void* combined,
                                    void* row_loss, unsigned int epoch,
                                    unsigned long long limit_ns, void* done_ctr, int* status,
                                    cudaStream_t st) {
  if (world > COMM_MAX_RANKS || T < 1) return -1;
  CommPeers c;
  fill_peers(c, bufs, flags, nullptr, rank, world);
  int grid = (T + 255) / 256;
  if (grid > 64) grid = 64;
  ce_stats_exchange_kernel<<<grid, 256, 0, st>>>(c, off, T, static_cast<const float*>(mask),
                                                 static_cast<float*>(combined),
                                                 static_cast<float*>(row_loss), epoch, limit_ns,
                                                 static_cast<unsigned int*>(done_ctr), status);
  return cudaGetLastError() == cudaSuccess ? 0 : -100;
}
