// Tensor-parallel GEMMs fused with their collective over NVLink peer memory (sm_100a).
// Same tcgen05 / TMEM / TMA pipeline as gemm_sm100.cu (bf16 in, fp32 accumulate, bf16 out),
// plus one of two communication roles inside the SAME kernel:
//
//  * all-gather -> GEMM  (column-parallel layers: QKV, gate/up, LM head, and the dgrads that
//    consume a gathered gradient). The A operand lives in a symmetric [M][K] buffer whose rows
//    are split in `tp` slots; this rank's slot is already written. Two extra warps per CTA pull
//    the peers' slots into the local buffer with plain 16-byte peer loads, 128-row chunk by
//    chunk, every CTA taking a slice of every chunk so a chunk lands after a few microseconds;
//    a per-chunk counter tells the TMA producer warp when a row block may be loaded. Tiles of
//    the local slot are scheduled first, so the tensor core starts at once and the transfer
//    hides behind it. A remote byte crosses NVLink once; TMA then reads local memory only.
//
//  * GEMM -> reduce-scatter  (row-parallel layers: O-proj, down-proj, and the dgrads of the
//    column-parallel layers). Each output tile is partial over the sharded reduction index and
//    belongs to the rank that owns its rows: the epilogue TMA-stores it straight into that
//    owner's `partials[src_rank]` plane (peer memory for remote owners). Remote-owned tiles
//    are scheduled first. The owner sums the `tp` planes in the consumer that follows
//    (tp_sum_partials_kernel below), so the reduction is deterministic and needs no atomics.
//
// Ranks synchronise with epoch flags in symmetric memory; every wait is bounded and reports
// through the status word. Stands in for the reference's NCCL all_reduce after / before its
// tensor-parallel GEMMs (exports/train_engine_8b/src/training_engine_tensor/forward.py:246,267;
// backward.py:454,580,725), restated as sequence-parallel all-gather / reduce-scatter.
#include <string.h>

#include "ptx.cuh"
#include "tma_host.h"

namespace ft {

int get_tmap_2d(CUtensorMap* out, const void* base, int elt, uint64_t rows, uint64_t cols,
                uint64_t ld, uint32_t box_r, uint32_t box_c);

constexpr int TP_BM = 128;
constexpr int TP_BK = 64;
constexpr int TP_BN = 256;
constexpr int TP_STAGES = 4;
constexpr int TP_THREADS = 320;  // warp 0 TMA, 1 MMA, 2-5 epilogue, 6-9 peer copy
constexpr int TP_COPY_THREADS = 128;
constexpr int TP_COPY_UNROLL = 8;
constexpr int TP_GROUP_M = 16;
constexpr int TP_MAX = 8;

struct TpGemmParams {
  int M, N, K;
  int b_mn;
  float alpha;
  int m_tiles, n_tiles, k_iters;
  int tp, rank, tiles_per_slot, slot_rows;
  int mode;               // 1: all-gather -> GEMM, 2: GEMM -> reduce-scatter
  // Work units [0, split_from) are whole 128 x 256 tiles; from split_from on, each tile of the
  // last, at most half-full wave is cut into two 128 x 128 halves (units 2i, 2i+1).
  int split_from, total_units;
  // all-gather side
  const uint8_t* a_peers[TP_MAX];  // peer base pointers of the gathered A buffer (own = local)
  long a_row_bytes;                // bytes per row (rows are contiguous)
  int* chunk_ready;                // [(tp-1) * tiles_per_slot] counters, zero at launch
  int copy_group;                  // CTAs that share one chunk (= arrivals expected per chunk)
  // flags / barriers
  uint32_t* flags[TP_MAX];         // peer flag arrays [8 slots][tp]
  uint32_t epoch;
  unsigned long long limit_ns;
  unsigned int* done_ctr;
  int* status;
};

struct TpSmem {
  static constexpr int A_BYTES = TP_BM * TP_BK * 2;
  static constexpr int B_BYTES = TP_BN * TP_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_BUF_BYTES = 4096;
  static constexpr int EPI_BYTES = 4 * 2 * EPI_BUF_BYTES;
  static constexpr int BAR_OFFSET = TP_STAGES * STAGE_BYTES + EPI_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;
};

__device__ __forceinline__ void tp_st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t tp_ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int tp_ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 tp_ld_peer16(const void* p) {
  uint4 v;
  asm volatile("ld.global.relaxed.sys.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Bounded wait on one peer flag (single thread). Returns false on time-out.
__device__ __forceinline__ bool tp_wait_flag(const uint32_t* f, uint32_t epoch, uint64_t limit_ns,
                                             int* status, volatile int* abort_flag) {
  const uint64_t t0 = globaltimer_ns();
  while (static_cast<int32_t>(tp_ld_acquire_sys(f) - epoch) < 0) {
    if (*abort_flag) return false;
    if (globaltimer_ns() - t0 > limit_ns) {
      *abort_flag = 1;
      if (status) atomicCAS(status, 0, FT_ERR_WAIT_PEER);
      return false;
    }
    __nanosleep(64);
  }
  return true;
}

// work unit -> (physical m tile, n tile, half). `rot` rotates the m order so that a rank starts
// with the row slot that needs no communication (mode 1) or ends with it (mode 2). `half`: -1
// for a whole tile, else which 128-column half of the tile this unit covers.
__device__ __forceinline__ void tp_decode_tile(const TpGemmParams& p, int tile, int rot, int& mt,
                                               int& nt, int& half) {
  half = -1;
  if (tile >= p.split_from) {
    const int t = tile - p.split_from;
    half = t & 1;
    tile = p.split_from + (t >> 1);
  }
  const int group_sz = TP_GROUP_M * p.n_tiles;
  const int g = tile / group_sz;
  const int first_m = g * TP_GROUP_M;
  const int gm = min(p.m_tiles - first_m, TP_GROUP_M);
  const int in = tile - g * group_sz;
  const int ml = first_m + in % gm;
  nt = in / gm;
  mt = (ml + rot) % p.m_tiles;
}

__global__ void __launch_bounds__(TP_THREADS, 1)
gemm_tp_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmD0, const __grid_constant__ CUtensorMap tmD1,
               const __grid_constant__ CUtensorMap tmD2, const __grid_constant__ CUtensorMap tmD3,
               const __grid_constant__ CUtensorMap tmD4, const __grid_constant__ CUtensorMap tmD5,
               const __grid_constant__ CUtensorMap tmD6, const __grid_constant__ CUtensorMap tmD7,
               const TpGemmParams p) {
  using L = TpSmem;
  constexpr int BN = TP_BN, STAGES = TP_STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* epi_base = smem + STAGES * L::STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_last = const_cast<int*>(reinterpret_cast<volatile int*>(tmem_slot + 2));

  const int warp = warp_idx_uniform();
  const int lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  const int rot = p.mode == 1 ? p.rank * p.tiles_per_slot
                              : ((p.rank + 1) % p.tp) * p.tiles_per_slot;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 4);
    }
    *abort_flag = 0;
    *s_last = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total_tiles = p.total_units;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    // One box per lane (lane 0: A, lanes 1..: B): a thread that issues a tiled TMA load is held
    // for several hundred cycles per instruction, so the boxes of a stage leave together.
    const int nB = p.b_mn ? BN / 64 : BN / 128;
    if (lane < 1 + nB) {
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        int mt, nt, half;
        tp_decode_tile(p, tile, rot, mt, nt, half);
        // a half tile loads only its half of the B boxes, into the start of the B buffer
        const int nBt = half < 0 ? nB : nB / 2;
        const int jb0 = half <= 0 ? 0 : nB / 2;
        const uint32_t tx = L::A_BYTES + (half < 0 ? L::B_BYTES : L::B_BYTES / 2);
        if (p.mode == 1 && lane == 0) {
          const int owner = mt / p.tiles_per_slot;
          if (owner != p.rank) {
            // wait until the CTAs that share this 128-row chunk have copied their slices
            const int hop = (owner - p.rank + p.tp) % p.tp;
            const int* ctr = p.chunk_ready + (hop - 1) * p.tiles_per_slot + mt % p.tiles_per_slot;
            const uint64_t t0 = globaltimer_ns();
            while (tp_ld_acquire_gpu(ctr) < p.copy_group) {
              if (*abort_flag) break;
              if (globaltimer_ns() - t0 > p.limit_ns) {
                *abort_flag = 1;
                if (p.status) atomicCAS(p.status, 0, FT_ERR_WAIT_PEER);
                break;
              }
            }
            // copies were generic-proxy stores; TMA reads through the async proxy
            asm volatile("fence.proxy.async.global;" ::: "memory");
          }
        }
        for (int ki = 0; ki < p.k_iters; ++ki) {
          mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, FT_ERR_WAIT_EMPTY);
          uint8_t* sA = smem + stage * L::STAGE_BYTES;
          uint8_t* sB = sA + L::A_BYTES;
          if (lane == 0) {
            // only this lane reads the gathered A operand, after its wait above
            mbar_expect_tx(&full_bar[stage], tx);
            tma_load_2d(sA, &tmA, &full_bar[stage], ki * TP_BK, mt * TP_BM);
          } else if (lane - 1 < nBt) {
            const int j = lane - 1;   // slot in the B buffer; jb0 + j: box of the tile
            if (!p.b_mn)
              tma_load_2d(sB + j * 16384, &tmB, &full_bar[stage], ki * TP_BK,
                          nt * BN + (jb0 + j) * 128);
            else
              tma_load_2d(sB + j * 8192, &tmB, &full_bar[stage], nt * BN + (jb0 + j) * 64,
                          ki * TP_BK);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (lane == 0 && *abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    // The whole warp walks the tiles and waits; one elected lane issues (see elect_one_sync).
    {
      const uint32_t idesc_full = make_idesc_bf16(TP_BM, BN, 0, p.b_mn);
      const uint32_t idesc_half = make_idesc_bf16(TP_BM, BN / 2, 0, p.b_mn);
      const uint32_t b_lbo = p.b_mn ? 8192u : 16u;
      const uint32_t b_kstep = p.b_mn ? (2048u >> 4) : (32u >> 4);
      const uint32_t smem_base = smem_u32(smem);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
        const uint32_t idesc = tile < p.split_from ? idesc_full : idesc_half;
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        mbar_wait(&tempty_bar[buf], acc_phase ^ 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_EMPTY);
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        for (int ki = 0; ki < p.k_iters; ++ki) {
          mbar_wait(&full_bar[stage], phase, abort_flag, p.status, FT_ERR_WAIT_FULL);
          tc_fence_after();
          if (elect_one_sync()) {
            const uint32_t sA = smem_base + stage * L::STAGE_BYTES;
            const uint32_t a_lo = smem_desc_lo(sA, 16);
            const uint32_t b_lo = smem_desc_lo(sA + L::A_BYTES, b_lbo);
            umma_ss_lo_dyn(tmem_d, a_lo, b_lo, idesc, ki > 0 ? 1u : 0u);
#pragma unroll
            for (int kk = 1; kk < TP_BK / 16; ++kk)
              umma_ss_lo<1>(tmem_d, a_lo + kk * 2, b_lo + kk * b_kstep, idesc);
            umma_commit(&empty_bar[stage]);
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (elect_one_sync()) umma_commit(&tfull_bar[buf]);
        __syncwarp();
      }
    }
  } else if (warp < 6) {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;
    uint8_t* my_epi = epi_base + q * 2 * L::EPI_BUF_BYTES;
    int it = 0, nstores = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
      int mt, nt, half;
      tp_decode_tile(p, tile, rot, mt, nt, half);
      const int ncols = half < 0 ? BN : BN / 2;
      const int colbase = nt * BN + (half > 0 ? BN / 2 : 0);
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      mbar_wait(&tfull_bar[buf], acc_phase, abort_flag, p.status, FT_ERR_WAIT_TMEM_FULL);
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
      const CUtensorMap* tmD = &tmD0;
      int row0 = mt * TP_BM + q * 32;
      int row_limit = p.M;
      if (p.mode == 2) {
        const int owner = mt / p.tiles_per_slot;
        tmD = owner == 0 ? &tmD0 : owner == 1 ? &tmD1 : owner == 2 ? &tmD2 : owner == 3 ? &tmD3
              : owner == 4 ? &tmD4 : owner == 5 ? &tmD5 : owner == 6 ? &tmD6 : &tmD7;
        row0 = (mt % p.tiles_per_slot) * TP_BM + q * 32;
        row_limit = p.slot_rows;
      }
      const bool rows_live = row0 < row_limit;
#pragma unroll 1
      for (int c = 0; c < ncols / 64; ++c) {
        const int col0 = colbase + c * 64;
        if (col0 >= p.N || !rows_live) break;
        uint32_t r[64];
        tmem_ld32(taddr + c * 64, r);
        tmem_ld32(taddr + c * 64 + 32, r + 32);
        tmem_ld_wait();
        uint8_t* sbuf = my_epi + (nstores & 1) * L::EPI_BUF_BYTES;
        if (nstores >= 2) {
          if (lane == 0) tma_wait_group_read<1>();
          __syncwarp();
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]) * p.alpha, __uint_as_float(r[8 * j + 1]) * p.alpha);
          v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]) * p.alpha, __uint_as_float(r[8 * j + 3]) * p.alpha);
          v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]) * p.alpha, __uint_as_float(r[8 * j + 5]) * p.alpha);
          v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]) * p.alpha, __uint_as_float(r[8 * j + 7]) * p.alpha);
          *reinterpret_cast<uint4*>(sbuf + lane * 128 + ((j ^ (lane & 7)) << 4)) = v;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(tmD, sbuf, col0, row0);
          tma_commit_group();
        }
        ++nstores;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
    }
    if (lane == 0) {
      tma_wait_group<0>();        // every store of this warp has been performed
      __threadfence_system();
    }
    __syncwarp();
  } else if (p.mode == 1) {
    // ------------------------------ peer copy warps (all-gather) ------------------------------
    const int ct = threadIdx.x - 6 * 32;  // 0..127
    // tell the peers that this rank's slot is complete (it was written before this launch)
    if (blockIdx.x == 0 && ct < p.tp && ct != p.rank) {
      __threadfence_system();
      tp_st_release_sys(p.flags[ct] + 0 * p.tp + p.rank, p.epoch);
    }
    uint8_t* local = const_cast<uint8_t*>(p.a_peers[p.rank]);
    // Chunks (128-row blocks of the peers' slots) are copied in parallel: a group of
    // `copy_group` CTAs shares one chunk, so every copy thread has dozens of independent
    // 16-byte peer loads to keep in flight and all chunks land at about the same time.
    const int n_chunks = (p.tp - 1) * p.tiles_per_slot;
    const int G = p.copy_group;
    int c_begin, c_step, part;
    if (G > 1 || n_chunks <= static_cast<int>(gridDim.x)) {
      c_begin = blockIdx.x / G;
      part = blockIdx.x % G;
      c_step = n_chunks;  // at most one chunk per CTA
    } else {
      c_begin = blockIdx.x;
      part = 0;
      c_step = gridDim.x;
    }
    int waited_src = -1;
    for (int c = c_begin; c < n_chunks; c += c_step) {
      const int hop = c / p.tiles_per_slot + 1;
      const int j = c % p.tiles_per_slot;
      const int src = (p.rank + hop) % p.tp;
      if (src != waited_src) {
        // one thread waits for the peer's "slot written" flag and publishes the outcome, so
        // that all copy threads take the same branch around the named barriers below
        if (ct == 0) {
          const bool ok = tp_wait_flag(p.flags[p.rank] + 0 * p.tp + src, p.epoch, p.limit_ns,
                                       p.status, abort_flag);
          s_last[1] = ok ? 1 : 0;
        }
        named_bar_sync(2, TP_COPY_THREADS);
        const int go = s_last[1];
        named_bar_sync(2, TP_COPY_THREADS);
        if (!go) break;
        waited_src = src;
      }
      const uint8_t* remote = p.a_peers[src];
      const long row_begin = static_cast<long>(src) * p.slot_rows + static_cast<long>(j) * TP_BM;
      long rows = p.slot_rows - static_cast<long>(j) * TP_BM;
      if (rows > TP_BM) rows = TP_BM;
      const long off = row_begin * p.a_row_bytes;
      const long nvec = rows * p.a_row_bytes / 16;
      const long per = (nvec + G - 1) / G;
      const long v0 = per * part;
      long v1 = v0 + per;
      if (v1 > nvec) v1 = nvec;
      for (long v = v0 + ct; v < v1; v += TP_COPY_THREADS * TP_COPY_UNROLL) {
        uint4 x[TP_COPY_UNROLL];
#pragma unroll
        for (int u = 0; u < TP_COPY_UNROLL; ++u)
          if (v + u * TP_COPY_THREADS < v1)
            x[u] = tp_ld_peer16(remote + off + (v + u * TP_COPY_THREADS) * 16);
#pragma unroll
        for (int u = 0; u < TP_COPY_UNROLL; ++u)
          if (v + u * TP_COPY_THREADS < v1)
            *reinterpret_cast<uint4*>(local + off + (v + u * TP_COPY_THREADS) * 16) = x[u];
      }
      __threadfence();
      named_bar_sync(2, TP_COPY_THREADS);
      if (ct == 0) atomicAdd(p.chunk_ready + c, 1);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  // exit barrier between ranks: mode 1 = "I no longer read your slot", mode 2 = "my partial
  // tiles are in your memory". The last CTA of this rank to get here signals and waits.
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int prev = atomicAdd(p.done_ctr, 1u);
    if (prev == gridDim.x - 1) {
      *s_last = 1;
      *p.done_ctr = 0;
    }
  }
  __syncthreads();
  if (*s_last) {
    const int slot = p.mode == 1 ? 1 : 2;
    if (threadIdx.x < p.tp && threadIdx.x != p.rank) {
      __threadfence_system();
      tp_st_release_sys(p.flags[threadIdx.x] + slot * p.tp + p.rank, p.epoch);
      tp_wait_flag(p.flags[p.rank] + slot * p.tp + threadIdx.x, p.epoch, p.limit_ns, p.status,
                   abort_flag);
    }
  }
}

// out[r][c] = bf16( sum_s partial[s][r][c] (+ res[r][c]) ), all bf16 storage, fp32 sum.
__global__ void __launch_bounds__(256)
tp_sum_partials_kernel(const __nv_bfloat16* __restrict__ partial, __nv_bfloat16* __restrict__ out,
                       long plane_elems, int tp) {
  const long nvec = plane_elems / 8;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    for (int s = 0; s < tp; ++s) {
      const uint4 v = reinterpret_cast<const uint4*>(partial + s * plane_elems)[i];
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        acc[2 * k] += bf16_lo(w[k]);
        acc[2 * k + 1] += bf16_hi(w[k]);
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

}  // namespace ft

using namespace ft;

static int tp_launch(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap* tD,
                     const TpGemmParams& p, int grid, cudaStream_t st) {
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(gemm_tp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             TpSmem::TOTAL) != cudaSuccess)
      return -10;
    attr = true;
  }
  gemm_tp_kernel<<<grid, TP_THREADS, TpSmem::TOTAL, st>>>(tA, tB, tD[0], tD[1], tD[2], tD[3], tD[4],
                                                          tD[5], tD[6], tD[7], p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

static int tp_grid() {
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms > 0 ? sms : 148;
}

// The all-gather -> GEMM grid waits on chunks that OTHER CTAs of the same grid bring in, so all
// of it has to be able to be resident at once: the launch is refused unless the device can hold
// `grid` CTAs of this kernel by itself. (Kernels of other streams can still delay single CTAs;
// they leave on their own, and every wait in the kernel is bounded.)
static bool tp_grid_fits(int grid) {
  static int per_sm = -1;
  if (per_sm < 0) {
    cudaFuncSetAttribute(gemm_tp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TpSmem::TOTAL);
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, gemm_tp_kernel, TP_THREADS,
                                                      TpSmem::TOTAL) != cudaSuccess)
      n = 0;
    per_sm = n;
  }
  return per_sm >= 1 && grid <= per_sm * tp_grid();
}

// Tail of the schedule, as in ft_gemm_bf16: when the last wave is at most half full, its tiles
// are cut into 128 x 128 halves on twice as many CTAs (a tensor-parallel rank of the 8B model at
// 4096 tokens has 512 tiles = 3.46 waves in the O-proj / FC2 forward and the QKV / FC1 dgrad).
static void tp_set_tail_split(TpGemmParams& p, int grid) {
  const int total = p.m_tiles * p.n_tiles;
  p.split_from = p.total_units = total;
  const int rem = total % grid;
  if (grid >= 2 && rem > 0 && 2 * rem <= grid) {
    p.split_from = total - rem;
    p.total_units = total + rem;
  }
}

// D[M,N] = alpha * gather(A)[M,K] * B^T. `a_peers[r]` is rank r's mapping of the symmetric
// gathered buffer ([M][K] bf16, contiguous rows); this rank's slot (rows rank*M/tp ..) holds
// its data, the other slots are filled by this call. B: [N][K] (b_mn = 0) or [K][N] (b_mn = 1)
// with leading dimension ldb. chunk_ready: (tp-1)*ceil(M/tp/128) ints (zeroed here).
// The grid must be fully co-resident (it is: one CTA per SM) because CTAs wait on one another.
extern "C" int ft_gemm_ag(const void* const* a_peers, const void* B, void* D, int M, int N, int K,
                          int ldb, int ldd, int b_mn, float alpha, int tp, int rank,
                          const void* const* flags, unsigned int epoch,
                          unsigned long long limit_ns, void* chunk_ready, void* done_ctr,
                          int* status, cudaStream_t st) {
  if (tp < 2 || tp > TP_MAX || M % tp || N < 1) return -1;
  const int slot_rows = M / tp;
  TpGemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K; p.b_mn = b_mn ? 1 : 0; p.alpha = alpha;
  p.m_tiles = (M + TP_BM - 1) / TP_BM;
  p.n_tiles = (N + TP_BN - 1) / TP_BN;
  p.k_iters = (K + TP_BK - 1) / TP_BK;
  if (slot_rows % TP_BM) return -2;  // row slots must be whole tiles
  p.tp = tp; p.rank = rank; p.tiles_per_slot = slot_rows / TP_BM; p.slot_rows = slot_rows;
  p.mode = 1;
  tp_set_tail_split(p, tp_grid());
  for (int i = 0; i < tp; ++i) {
    p.a_peers[i] = static_cast<const uint8_t*>(a_peers[i]);
    p.flags[i] = static_cast<uint32_t*>(const_cast<void*>(flags[i]));
  }
  p.a_row_bytes = static_cast<long>(K) * 2;
  p.chunk_ready = static_cast<int*>(chunk_ready);
  p.epoch = epoch; p.limit_ns = limit_ns;
  p.done_ctr = static_cast<unsigned int*>(done_ctr);
  p.status = status;
  const int grid = tp_grid();
  if (!tp_grid_fits(grid)) return -7;
  const int n_chunks = (tp - 1) * p.tiles_per_slot;
  p.copy_group = n_chunks <= grid ? grid / n_chunks : 1;
  if (cudaMemsetAsync(chunk_ready, 0, sizeof(int) * n_chunks, st) != cudaSuccess) return -3;
  CUtensorMap tA, tB, tD[8];
  if (get_tmap_2d(&tA, a_peers[rank], 2, M, K, K, TP_BM, TP_BK)) return -4;
  int rc = b_mn ? get_tmap_2d(&tB, B, 2, K, N, ldb, TP_BK, 64) : get_tmap_2d(&tB, B, 2, N, K, ldb, 128, TP_BK);
  if (rc) return -5;
  if (get_tmap_2d(&tD[0], D, 2, M, N, ldd, 32, 64)) return -6;
  for (int i = 1; i < 8; ++i) tD[i] = tD[0];
  return tp_launch(tA, tB, tD, p, grid, st);
}

// partial planes: every rank owns `partials` = [tp][M/tp][N] bf16 in symmetric memory;
// `d_peers[o]` is owner o's mapping of it. This rank's tile rows that belong to owner o are
// stored into plane `rank` of owner o. After the call (kernel end) this rank's own planes hold
// every rank's contribution for its row slot; sum them with ft_tp_sum_partials.
extern "C" int ft_gemm_rs(const void* A, const void* B, const void* const* d_peers, int M, int N,
                          int K, int lda, int ldb, int b_mn, float alpha, int tp, int rank,
                          const void* const* flags, unsigned int epoch,
                          unsigned long long limit_ns, void* done_ctr, int* status,
                          cudaStream_t st) {
  if (tp < 2 || tp > TP_MAX || M % tp) return -1;
  const int slot_rows = M / tp;
  if (slot_rows % TP_BM) return -2;
  TpGemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K; p.b_mn = b_mn ? 1 : 0; p.alpha = alpha;
  p.m_tiles = (M + TP_BM - 1) / TP_BM;
  p.n_tiles = (N + TP_BN - 1) / TP_BN;
  p.k_iters = (K + TP_BK - 1) / TP_BK;
  p.tp = tp; p.rank = rank; p.tiles_per_slot = slot_rows / TP_BM; p.slot_rows = slot_rows;
  p.mode = 2;
  tp_set_tail_split(p, tp_grid());
  for (int i = 0; i < tp; ++i) p.flags[i] = static_cast<uint32_t*>(const_cast<void*>(flags[i]));
  p.epoch = epoch; p.limit_ns = limit_ns;
  p.done_ctr = static_cast<unsigned int*>(done_ctr);
  p.status = status;
  CUtensorMap tA, tB, tD[8];
  if (get_tmap_2d(&tA, A, 2, M, K, lda, TP_BM, TP_BK)) return -4;
  int rc = b_mn ? get_tmap_2d(&tB, B, 2, K, N, ldb, TP_BK, 64) : get_tmap_2d(&tB, B, 2, N, K, ldb, 128, TP_BK);
  if (rc) return -5;
  for (int o = 0; o < 8; ++o) {
    const int oo = o < tp ? o : 0;
    const __nv_bfloat16* base = static_cast<const __nv_bfloat16*>(d_peers[oo]) +
                                static_cast<long>(rank) * slot_rows * N;
    if (get_tmap_2d(&tD[o], base, 2, slot_rows, N, N, 32, 64)) return -6;
  }
  return tp_launch(tA, tB, tD, p, tp_grid(), st);
}

extern "C" int ft_tp_sum_partials(const void* partial, void* out, long plane_elems, int tp,
                                  cudaStream_t st) {
  if (plane_elems % 8) return -1;
  long blocks = (plane_elems / 8 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  tp_sum_partials_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(partial), static_cast<__nv_bfloat16*>(out), plane_elems, tp);
  return cudaGetLastError() == cudaSuccess ? 0 : -100;
}
