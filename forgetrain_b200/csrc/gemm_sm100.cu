// Persistent, warp-specialised bf16 GEMM for sm_100a:
//   D[M,N] (=|+=) alpha * sum_k A[m,k] * B[n,k]
// * operands are staged by TMA (128-byte swizzle, one CTA per load) into a multi-stage ring
//   by two producer warps, several lanes each (one box per lane),
// * one thread issues tcgen05.mma (128 x BN x 16 per instruction) into TMEM accumulators,
// * two accumulator buffers in TMEM let the epilogue of tile i overlap the main loop of
//   tile i+1,
// * the epilogue reads TMEM with tcgen05.ld, converts, stages through swizzled shared memory
//   and leaves through TMA stores (bf16 / fp32) or TMA reduce-adds (fp32 accumulate, which
//   is also what makes split-K need no separate reduction pass).
// Both operands may be K-major (reduction index contiguous) or MN-major (row index
// contiguous), so forward (x W^T), dgrad (dy W) and wgrad (dy^T x) all run on this kernel
// without any transposed copy. Row / column / reduction tails are handled by TMA
// out-of-bounds fill and clipping, so no padded copies are needed either.
//
// Covers the role of the reference's per-projection GEMM kernels and their launchers
// (ops/gemm_fc1/gemm_sm90.cu, ops/gemm_*/gemm_cutedsl.cpp, ops/gemm_qkv_proj/_aot_reduce.cu).
#include <mutex>
#include <unordered_map>
#include <string>
#include <string.h>
#include <stdlib.h>

#include "ptx.cuh"
#include "swiglu_math.cuh"
#include "tma_host.h"

namespace ft {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
// warps 0 and 10: TMA producers (even / odd stages), warp 1: MMA + TMEM owner, warps 2-9: epilogue.
// A thread that issues a tiled TMA load is held for roughly 400 cycles per instruction whatever
// the box size, so one issuing thread cannot feed a 500-cycle k-step that needs two or more
// boxes; the boxes of a stage are therefore issued by different lanes of one instruction and
// alternate stages by different warps.
constexpr int GEMM_THREADS = 352;
constexpr int GEMM_PRODUCER_WARP2 = 10;
constexpr int GEMM_EPI_WARPS = 8;    // two warps per TMEM lane quarter, each takes half the columns
constexpr int GEMM_GROUP_M = 16;

enum : int { OUT_BF16 = 0, OUT_F32 = 1, OUT_F32_ADD = 2 };
// what the epilogue does besides scaling and storing the accumulator
enum : int { EPI_PLAIN = 0, EPI_SWIGLU_FWD = 1, EPI_SWIGLU_BWD = 2 };

struct GemmParams {
  int M, N, K;
  int a_mn, b_mn;     // 1: operand is MN-major
  int out_mode;       // OUT_*
  float alpha;
  int splitk;
  int m_tiles, n_tiles, k_iters;
  int* status;
  int swiglu_F;       // > 0 (EPI_SWIGLU_FWD): B is [2F][K] = [gate rows ; up rows];
                      //     (EPI_SWIGLU_BWD): N == F, D is [M][2F] = [d gate ; d up]
  // Work units [0, split_from) are whole 128 x BN tiles; from split_from on, each tile of the
  // last, partly filled wave is cut into two 128 x BN/2 halves (units 2i, 2i+1), so that the
  // tail of the schedule costs about 0.6 instead of 1.0 tile times. total_units counts both.
  int split_from, total_units;
};

template <int BN, int STAGES, int EPI_BUFS = 1>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_BUF_BYTES = 4096 * EPI_BUFS;      // boxes of 32 rows x 128 B
  static constexpr int EPI_BYTES = GEMM_EPI_WARPS * EPI_BUF_BYTES;  // one buffer per warp
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES + EPI_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 512 + 1024;      // + barriers + alignment slack
};

// `half`: -1 for a whole tile, else which half of the tile's columns this unit covers.
__device__ __forceinline__ void decode_tile(const GemmParams& p, int tile, int& mt, int& nt,
                                            int& kb, int& kn, int& half) {
  half = -1;
  if (tile >= p.split_from) {
    const int t = tile - p.split_from;
    half = t & 1;
    tile = p.split_from + (t >> 1);
  }
  const int per_split = p.m_tiles * p.n_tiles;
  const int ks = tile / per_split;
  const int r = tile - ks * per_split;
  const int group_sz = GEMM_GROUP_M * p.n_tiles;
  const int g = r / group_sz;
  const int first_m = g * GEMM_GROUP_M;
  const int gm = min(p.m_tiles - first_m, GEMM_GROUP_M);
  const int in = r - g * group_sz;
  mt = first_m + in % gm;
  nt = in / gm;
  const int base = p.k_iters / p.splitk, rem = p.k_iters % p.splitk;
  kb = ks * base + min(ks, rem);
  kn = base + (ks < rem ? 1 : 0);
}

// Epilogue of one 128 x ncols accumulator for one warp: its 32 TMEM lanes (rows row0..row0+31),
// column half `chalf`. TMEM -> registers -> (alpha, convert) -> swizzled staging buffer ->
// TMA store / reduce-add. `nstores` counts this warp's bulk groups so the staging buffer is
// only rewritten after the previous store has read it.
__device__ __forceinline__ void drain_tile(const GemmParams& p, const CUtensorMap* tmD,
                                           uint32_t taddr, int row0, int colbase, int ncols,
                                           int chalf, uint8_t* sbuf, int lane, int& nstores) {
  const bool rows_live = row0 < p.M;
  if (p.out_mode == OUT_BF16) {
#pragma unroll 1
    for (int c = chalf * (ncols / 128); c < (chalf + 1) * (ncols / 128); ++c) {
      const int col0 = colbase + c * 64;
      if (col0 >= p.N || !rows_live) break;
      uint32_t r[64];
      tmem_ld32(taddr + c * 64, r);
      tmem_ld32(taddr + c * 64 + 32, r + 32);
      tmem_ld_wait();
      if (nstores >= 1) {
        if (lane == 0) tma_wait_group_read<0>();
        __syncwarp();
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint4 v;
        v.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]) * p.alpha,
                          __uint_as_float(r[8 * j + 1]) * p.alpha);
        v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]) * p.alpha,
                          __uint_as_float(r[8 * j + 3]) * p.alpha);
        v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]) * p.alpha,
                          __uint_as_float(r[8 * j + 5]) * p.alpha);
        v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]) * p.alpha,
                          __uint_as_float(r[8 * j + 7]) * p.alpha);
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
  } else {
#pragma unroll 1
    for (int c = chalf * (ncols / 64); c < (chalf + 1) * (ncols / 64); ++c) {
      const int col0 = colbase + c * 32;
      if (col0 >= p.N || !rows_live) break;
      uint32_t r[32];
      tmem_ld32(taddr + c * 32, r);
      tmem_ld_wait();
      if (nstores >= 1) {
        if (lane == 0) tma_wait_group_read<0>();
        __syncwarp();
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 v;
        v.x = __uint_as_float(r[4 * j + 0]) * p.alpha;
        v.y = __uint_as_float(r[4 * j + 1]) * p.alpha;
        v.z = __uint_as_float(r[4 * j + 2]) * p.alpha;
        v.w = __uint_as_float(r[4 * j + 3]) * p.alpha;
        *reinterpret_cast<float4*>(sbuf + lane * 128 + ((j ^ (lane & 7)) << 4)) = v;
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        if (p.out_mode == OUT_F32_ADD)
          tma_reduce_add_2d(tmD, sbuf, col0, row0);
        else
          tma_store_2d(tmD, sbuf, col0, row0);
        tma_commit_group();
      }
      ++nstores;
    }
  }
}

// Epilogue of the fused FC1 + SwiGLU tile. The accumulator's columns 0..127 are gate columns
// n0..n0+127 and its columns 128..255 the up columns F+n0..F+n0+127 of the same rows. A warp
// takes 64 gate columns and the matching 64 up columns, writes both (bf16) into Y, which the
// backward pass reads, and act = silu(gate) * up into ACT. The activation is computed from the
// ROUNDED bf16 gate / up values with the arithmetic of swiglu_fwd_kernel, so it is bitwise the
// result of running that kernel on Y.
__device__ __forceinline__ void drain_tile_swiglu(const GemmParams& p, const CUtensorMap* tmY,
                                                  const CUtensorMap* tmAct, uint32_t taddr,
                                                  int row0, int n0, int chalf, uint8_t* sbuf,
                                                  int lane, int& nstores) {
  if (row0 >= p.M) return;
  const int gcol = n0 + chalf * 64;
  if (gcol >= p.swiglu_F) return;
  // Three 64-column stores go through the warp's one staging buffer, each waiting until the
  // previous store has read it. The TMEM load of the up half and the activation arithmetic are
  // placed between the stores so that they run during those reads.
  uint32_t g[32], u[32];   // 64 gate and 64 up values of this thread's row, packed bf16x2
  uint32_t r[64];
  auto put = [&](const uint32_t* w, const CUtensorMap* tm, int col) {
    if (nstores >= 1) {
      if (lane == 0) tma_wait_group_read<0>();
      __syncwarp();
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
      *reinterpret_cast<uint4*>(sbuf + lane * 128 + ((j ^ (lane & 7)) << 4)) =
          make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(tm, sbuf, col, row0);
      tma_commit_group();
    }
    ++nstores;
  };
  tmem_ld32(taddr + chalf * 64, r);
  tmem_ld32(taddr + chalf * 64 + 32, r + 32);
  tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 32; ++i)
    g[i] = pack_bf16x2(__uint_as_float(r[2 * i]) * p.alpha, __uint_as_float(r[2 * i + 1]) * p.alpha);
  tmem_ld32(taddr + 128 + chalf * 64, r);
  tmem_ld32(taddr + 128 + chalf * 64 + 32, r + 32);
  put(g, tmY, gcol);
  tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 32; ++i)
    u[i] = pack_bf16x2(__uint_as_float(r[2 * i]) * p.alpha, __uint_as_float(r[2 * i + 1]) * p.alpha);
  put(u, tmY, p.swiglu_F + gcol);
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const uint32_t gw = g[i], uw = u[i];
    const float g0 = __uint_as_float(gw << 16), g1 = __uint_as_float(gw & 0xffff0000u);
    const float u0 = __uint_as_float(uw << 16), u1 = __uint_as_float(uw & 0xffff0000u);
    const float s0 = 1.f / (1.f + __expf(-g0)), s1 = 1.f / (1.f + __expf(-g1));
    g[i] = pack_bf16x2(g0 * s0 * u0, g1 * s1 * u1);
  }
  put(g, tmAct, gcol);
}

// Epilogue of the fused FC2 dgrad + SwiGLU backward kernel (EPI_SWIGLU_BWD), one warp's share.
// The accumulator holds d act = alpha * dY W2 for 256 (or 128) columns of F; the warp owns 32 rows
// and half of the columns and walks them in pieces of 32 columns. For every piece the gate box and
// the up box (32 rows x 32 columns, bf16) of the FC1 output of the forward pass come into one of
// two staging sets by TMA, every thread reads its own row of both, and d gate / d up go back out
// through the same set into D[M][2F]; the [M][F] gradient of the activation never goes to memory.
// The loads of piece i+1 (which may belong to the next tile) are issued while piece i is being
// computed, so their latency is hidden. (Row-owner threads reading their rows straight from
// global memory touch 32 different lines per instruction; that ran at a tenth of the memory
// bandwidth.) d act is rounded to bf16 first and the arithmetic is swiglu_bwd_elem, so the result
// is bitwise what the dgrad GEMM followed by swiglu_bwd_kernel produces.
struct SwigluBwdCursor {   // position of the load look-ahead in this warp's list of pieces
  int tile, sub, nvalid, row0, col0;
};

template <int BN>
__device__ __forceinline__ void swiglu_bwd_tile_info(const GemmParams& p, int tile, int q,
                                                     int chalf, int& row0, int& col0, int& ncols,
                                                     int& nvalid) {
  int mt, nt, kb, kn, half;
  decode_tile(p, tile, mt, nt, kb, kn, half);
  ncols = half < 0 ? BN : BN / 2;
  row0 = mt * GEMM_BM + q * 32;
  col0 = nt * BN + (half > 0 ? BN / 2 : 0) + chalf * (ncols / 2);
  // F is a multiple of 64, so a 32-column piece is inside or outside as a whole
  const int left = (p.swiglu_F - col0) / 32;
  nvalid = row0 < p.M ? max(0, min(ncols / 64, left)) : 0;
}

template <int BN, int STAGES, int EPI = EPI_PLAIN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmD2,
                 const GemmParams p) {
  constexpr bool SWIGLU = EPI == EPI_SWIGLU_FWD;
  static_assert(EPI == EPI_PLAIN || BN == 256, "the fused SwiGLU epilogues are built for 256-column tiles");
  using L = GemmSmem<BN, STAGES, EPI == EPI_SWIGLU_BWD ? 2 : 1>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* epi_base = smem + STAGES * L::STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint64_t* ybar = tempty_bar + 2;   // EPI_SWIGLU_BWD: two per epilogue warp (gate / up boxes landed)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ybar + 2 * GEMM_EPI_WARPS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = warp_idx_uniform();
  const int lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 2 * BN;  // 256 or 512: two fp32 accumulators of BN columns

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], GEMM_EPI_WARPS);
    }
    for (int w = 0; w < 2 * GEMM_EPI_WARPS; ++w) mbar_init(&ybar[w], 1);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    prefetch_tmap(&tmD);
    if (EPI != EPI_PLAIN) prefetch_tmap(&tmD2);
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

  if (warp == 0 || warp == GEMM_PRODUCER_WARP2) {
    // ------------------------------ TMA producers ------------------------------
    // Lane l issues box l of a stage: A is one 128-row box (K-major) or two 64 x 64 boxes
    // (MN-major); B is BN/128 boxes of 128 rows or BN/64 boxes of 64 x 64.
    const int pid = warp == 0 ? 0 : 1;
    const int nA = p.a_mn ? GEMM_BM / 64 : 1;
    const int nB = p.b_mn ? BN / 64 : BN / 128;
    if (lane < nA + nB) {
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        int mt, nt, kb, kn, half;
        decode_tile(p, tile, mt, nt, kb, kn, half);
        // a half tile loads only its half of the B boxes, into the start of the B buffer
        const int nBt = half < 0 ? nB : nB / 2;
        const int jb0 = half <= 0 ? 0 : nB / 2;
        const uint32_t tx = L::A_BYTES + (half < 0 ? L::B_BYTES : L::B_BYTES / 2);
        for (int ki = kb; ki < kb + kn; ++ki) {
          if ((stage & 1) == pid) {
            mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, FT_ERR_WAIT_EMPTY);
            uint8_t* sA = smem + stage * L::STAGE_BYTES;
            uint8_t* sB = sA + L::A_BYTES;
            if (lane == 0) mbar_expect_tx(&full_bar[stage], tx);
            if (lane < nA) {
              if (!p.a_mn)
                tma_load_2d(sA, &tmA, &full_bar[stage], ki * GEMM_BK, mt * GEMM_BM);
              else
                tma_load_2d(sA + lane * 8192, &tmA, &full_bar[stage], mt * GEMM_BM + lane * 64,
                            ki * GEMM_BK);
            } else if (lane - nA < nBt) {
              const int j = lane - nA;           // slot in the B buffer; jb0 + j: box of the tile
              if (SWIGLU)   // box 0: 128 gate rows, box 1: the 128 up rows of the same columns
                tma_load_2d(sB + j * 16384, &tmB, &full_bar[stage], ki * GEMM_BK,
                            nt * 128 + j * p.swiglu_F);
              else if (!p.b_mn)
                tma_load_2d(sB + j * 16384, &tmB, &full_bar[stage], ki * GEMM_BK,
                            nt * BN + (jb0 + j) * 128);
              else
                tma_load_2d(sB + j * 8192, &tmB, &full_bar[stage], nt * BN + (jb0 + j) * 64,
                            ki * GEMM_BK);
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      // Tail: observe the release of every stage once more, so that no asynchronous arrival of
      // the tensor pipe is still on its way when the CTA exits.
      for (int i = 0; i < STAGES; ++i) {
        if ((stage & 1) == pid)
          mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, FT_ERR_WAIT_EMPTY);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
      if (lane == 0 && *abort_flag) {
        // Give copies still in flight time to land before the CTA's shared memory goes away.
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    // The whole warp walks the tiles and waits on the barriers; one elected lane issues, so
    // that descriptors, TMEM addresses and loop state stay warp-uniform (see elect_one_sync).
    {
      const uint32_t idesc_full = make_idesc_bf16(GEMM_BM, BN, p.a_mn, p.b_mn);
      const uint32_t idesc_half = make_idesc_bf16(GEMM_BM, BN / 2, p.a_mn, p.b_mn);
      const uint32_t a_lbo = p.a_mn ? 8192u : 16u, b_lbo = p.b_mn ? 8192u : 16u;
      const uint32_t a_kstep = p.a_mn ? (2048u >> 4) : (32u >> 4);
      const uint32_t b_kstep = p.b_mn ? (2048u >> 4) : (32u >> 4);
      const uint32_t smem_base = smem_u32(smem);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
        int mt, nt, kb, kn, half;
        decode_tile(p, tile, mt, nt, kb, kn, half);
        const uint32_t idesc = half < 0 ? idesc_full : idesc_half;
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        mbar_wait(&tempty_bar[buf], acc_phase ^ 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_EMPTY);
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        for (int ki = 0; ki < kn; ++ki) {
          mbar_wait(&full_bar[stage], phase, abort_flag, p.status, FT_ERR_WAIT_FULL);
          tc_fence_after();
          if (elect_one_sync()) {
            const uint32_t sA = smem_base + stage * L::STAGE_BYTES;
            const uint32_t a_lo = smem_desc_lo(sA, a_lbo);
            const uint32_t b_lo = smem_desc_lo(sA + L::A_BYTES, b_lbo);
            umma_ss_lo_dyn(tmem_d, a_lo, b_lo, idesc, ki > 0 ? 1u : 0u);
#pragma unroll
            for (int kk = 1; kk < GEMM_BK / 16; ++kk)
              umma_ss_lo<1>(tmem_d, a_lo + kk * a_kstep, b_lo + kk * b_kstep, idesc);
            umma_commit(&empty_bar[stage]);
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (elect_one_sync()) umma_commit(&tfull_bar[buf]);
        __syncwarp();
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;             // TMEM lane quarter this warp may access
    const int chalf = (warp - 2) >> 2;  // which half of the tile's columns this warp drains
    uint8_t* my_epi = epi_base + (warp - 2) * L::EPI_BUF_BYTES;
    int it = 0;
    int nstores = 0;
    if constexpr (EPI == EPI_SWIGLU_BWD) {
      uint64_t* yb = &ybar[(warp - 2) * 2];   // loads of staging set 0 / 1 have landed
      const int total = total_tiles;
      auto advance = [&](SwigluBwdCursor& c) {   // to the next piece that exists
        ++c.sub;
        while (c.tile < total && c.sub >= c.nvalid) {
          c.tile += gridDim.x;
          c.sub = 0;
          if (c.tile < total) {
            int nc;
            swiglu_bwd_tile_info<BN>(p, c.tile, q, chalf, c.row0, c.col0, nc, c.nvalid);
          }
        }
      };
      auto issue = [&](const SwigluBwdCursor& c, int set) {   // lane 0 only
        uint8_t* dst = my_epi + set * 4096;
        mbar_expect_tx(&yb[set], 4096);
        tma_load_2d(dst, &tmD2, &yb[set], c.col0 + c.sub * 32, c.row0);
        tma_load_2d(dst + 2048, &tmD2, &yb[set], p.swiglu_F + c.col0 + c.sub * 32, c.row0);
      };
      SwigluBwdCursor la;
      la.tile = blockIdx.x;
      la.sub = -1;
      la.nvalid = 0;
      if (la.tile < total) {
        int nc;
        swiglu_bwd_tile_info<BN>(p, la.tile, q, chalf, la.row0, la.col0, nc, la.nvalid);
      }
      advance(la);
      if (la.tile < total) {   // the first piece's boxes: on their way before the first accumulator
        if (lane == 0) issue(la, 0);
        advance(la);
      }
      uint32_t nitem = 0;
      for (int tile = blockIdx.x; tile < total; tile += gridDim.x, ++it) {
        int row0, col0, ncols, nvalid;
        swiglu_bwd_tile_info<BN>(p, tile, q, chalf, row0, col0, ncols, nvalid);
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        mbar_wait(&tfull_bar[buf], acc_phase, abort_flag, p.status, FT_ERR_WAIT_TMEM_FULL);
        tc_fence_after();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN +
                               chalf * (ncols / 2);
        if (tile + static_cast<int>(gridDim.x) < total) {
          // the boxes of this warp's pieces of the NEXT tile go to L2 a tile time ahead
          int r2, c2, nc2, nv2;
          swiglu_bwd_tile_info<BN>(p, tile + gridDim.x, q, chalf, r2, c2, nc2, nv2);
          if (lane < 2 * nv2)
            tma_prefetch_l2_2d(&tmD2, c2 + (lane >> 1) * 32 + (lane & 1) * p.swiglu_F, r2);
        }
#pragma unroll 1
        for (int sub = 0; sub < nvalid; ++sub, ++nitem) {
          const int set = nitem & 1;
          uint8_t* const bufG = my_epi + set * 4096;
          uint8_t* const bufU = bufG + 2048;
          // this row's 32 accumulator values, scaled and rounded to bf16
          uint32_t d[16];
          {
            uint32_t r[32];
            tmem_ld32(taddr + sub * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i)
              d[i] = pack_bf16x2(__uint_as_float(r[2 * i]) * p.alpha,
                                 __uint_as_float(r[2 * i + 1]) * p.alpha);
          }
          mbar_wait(&yb[set], (nitem >> 1) & 1, abort_flag, p.status, FT_ERR_WAIT_FULL);
          // 64-byte rows under the 64-byte swizzle: 16-byte piece j of row r sits at piece
          // j ^ ((r / 2) % 4) of the row (address bits 4-5 xor bits 7-8)
          uint32_t g[16], u[16];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int off = lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4);
            const uint4 gv = *reinterpret_cast<const uint4*>(bufG + off);
            const uint4 uv = *reinterpret_cast<const uint4*>(bufU + off);
            g[4 * j] = gv.x; g[4 * j + 1] = gv.y; g[4 * j + 2] = gv.z; g[4 * j + 3] = gv.w;
            u[4 * j] = uv.x; u[4 * j + 1] = uv.y; u[4 * j + 2] = uv.z; u[4 * j + 3] = uv.w;
          }
          // the other set: free once the previous piece's stores have read it; the next piece's
          // boxes start now and land while this piece is computed
          if (la.tile < total) {
            if (lane == 0) {
              if (nstores >= 1) tma_wait_group_read<0>();
              issue(la, set ^ 1);
            }
            advance(la);
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float d0 = __uint_as_float(d[i] << 16), d1 = __uint_as_float(d[i] & 0xffff0000u);
            const float g0 = __uint_as_float(g[i] << 16), g1 = __uint_as_float(g[i] & 0xffff0000u);
            const float u0 = __uint_as_float(u[i] << 16), u1 = __uint_as_float(u[i] & 0xffff0000u);
            float dg0, du0, dg1, du1;
            swiglu_bwd_elem(d0, g0, u0, dg0, du0);
            swiglu_bwd_elem(d1, g1, u1, dg1, du1);
            g[i] = pack_bf16x2(dg0, dg1);
            u[i] = pack_bf16x2(du0, du1);
          }
          __syncwarp();   // every lane has read its rows: the set may be overwritten
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int off = lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4);
            *reinterpret_cast<uint4*>(bufG + off) =
                make_uint4(g[4 * j], g[4 * j + 1], g[4 * j + 2], g[4 * j + 3]);
            *reinterpret_cast<uint4*>(bufU + off) =
                make_uint4(u[4 * j], u[4 * j + 1], u[4 * j + 2], u[4 * j + 3]);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmD, bufG, col0 + sub * 32, row0);
            tma_store_2d(&tmD, bufU, p.swiglu_F + col0 + sub * 32, row0);
            tma_commit_group();
          }
          ++nstores;
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[buf]);
      }
    } else {
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
      int mt, nt, kb, kn, half;
      decode_tile(p, tile, mt, nt, kb, kn, half);
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      mbar_wait(&tfull_bar[buf], acc_phase, abort_flag, p.status, FT_ERR_WAIT_TMEM_FULL);
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
      const int row0 = mt * GEMM_BM + q * 32;
      if (SWIGLU)
        drain_tile_swiglu(p, &tmD, &tmD2, taddr, row0, nt * 128, chalf, my_epi, lane, nstores);
      else
        drain_tile(p, &tmD, taddr, row0, nt * BN + (half > 0 ? BN / 2 : 0),
                   half < 0 ? BN : BN / 2, chalf, my_epi, lane, nstores);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
    }
    }
    if (lane == 0) tma_wait_group<0>();
    __syncwarp();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

#ifdef FT_BUILD_PAIR_GEMM
// ---------------------------------------------------------------------------------------
// CTA-pair variant (NOT BUILT: kept for reading only, behind FT_BUILD_PAIR_GEMM, which the
// build never defines; under neighbour load on a shared GPU this kernel stopped making progress
// and the cause has not been found): a cluster of two CTAs owns a 256 x 256 output tile. Each CTA stages 128
// rows of A and 128 columns' worth of B per k-step (32 KB instead of 48 KB for 128 x 256 of
// output), so shared-memory write (TMA) plus read (tensor core) traffic per SM drops by a
// third and six stages fit. The even CTA issues every MMA (`cta_group::2`, M = 256); each CTA
// drains the 128 accumulator rows that live in its own TMEM.
//   full[s]   (even CTA)  : armed by the even CTA's producer with both CTAs' bytes; both CTAs'
//                           loads report to it.
//   empty[s]  (each CTA)  : one commit from the issuing thread signals the barrier of both
//                           CTAs (a second commit instruction per stage, or a relayed
//                           arrive, measurably stalls the pipe).
//   tfull[b]  (each CTA)  : same, at the end of a tile.
//   tempty[b] (even CTA)  : 16 arrivals, one per epilogue warp of both CTAs.
// ---------------------------------------------------------------------------------------
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_BN = 256;
struct PairSmem {
  static constexpr int A_BYTES = 128 * GEMM_BK * 2;
  static constexpr int B_BYTES = 128 * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_BUF_BYTES = 4096;
  static constexpr int EPI_BYTES = GEMM_EPI_WARPS * EPI_BUF_BYTES;
  static constexpr int BAR_OFFSET = PAIR_STAGES * STAGE_BYTES + EPI_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_pair_bf16_kernel(const __grid_constant__ CUtensorMap tmA,
                      const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmD, const GemmParams p) {
  using L = PairSmem;
  constexpr int STAGES = PAIR_STAGES;
  constexpr int BN = PAIR_BN;
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

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  constexpr uint32_t TMEM_COLS = 2 * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 2 * GEMM_EPI_WARPS);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    prefetch_tmap(&tmD);
  }
  __syncwarp();
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the peer's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int total_tiles = p.m_tiles * p.n_tiles * p.splitk;
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

  if (warp == 0 || warp == GEMM_PRODUCER_WARP2) {
    // ------------------------------ TMA producers (both CTAs) ------------------------------
    const int pid = warp == 0 ? 0 : 1;
    const int nA = p.a_mn ? 2 : 1;
    const int nB = p.b_mn ? 2 : 1;
    if (lane < nA + nB) {
      const uint32_t full0 = mapa_u32(smem_u32(&full_bar[0]), 0);
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = pair; tile < total_tiles; tile += npairs) {
        int mt, nt, kb, kn;
        int half_unused; decode_tile(p, tile, mt, nt, kb, kn, half_unused);
        const int arow = mt * 256 + static_cast<int>(rank) * 128;
        const int brow = nt * BN + static_cast<int>(rank) * 128;
        for (int ki = kb; ki < kb + kn; ++ki) {
          if ((stage & 1) == pid) {
            mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, FT_ERR_WAIT_EMPTY);
            uint8_t* sA = smem + stage * L::STAGE_BYTES;
            uint8_t* sB = sA + L::A_BYTES;
            if (leader && lane == 0) mbar_expect_tx(&full_bar[stage], 2 * L::STAGE_BYTES);
            const uint32_t bar = full0 + stage * 8;
            if (lane < nA) {
              if (!p.a_mn)
                tma_load_2d_pair(sA, &tmA, bar, ki * GEMM_BK, arow);
              else
                tma_load_2d_pair(sA + lane * 8192, &tmA, bar, arow + lane * 64, ki * GEMM_BK);
            } else {
              const int j = lane - nA;
              if (!p.b_mn)
                tma_load_2d_pair(sB, &tmB, bar, ki * GEMM_BK, brow);
              else
                tma_load_2d_pair(sB + j * 8192, &tmB, bar, brow + j * 64, ki * GEMM_BK);
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      // Tail: one more trip round the ring, waiting only. The releases of the last stages are
      // asynchronous arrivals sent by the other CTA's tensor pipe; each of them has to be
      // observed here before this CTA may exit, or it would land in the shared memory of
      // whatever CTA (of any kernel) gets this SM next.
      for (int i = 0; i < STAGES; ++i) {
        if ((stage & 1) == pid)
          mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, FT_ERR_WAIT_EMPTY);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
      if (lane == 0 && *abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (even CTA only) ------------------------------
    if (lane == 0 && leader) {
      const uint32_t idesc = make_idesc_bf16(256, BN, p.a_mn, p.b_mn);
      const uint32_t a_lbo = p.a_mn ? 8192u : 16u, b_lbo = p.b_mn ? 8192u : 16u;
      const uint32_t a_kstep = p.a_mn ? (2048u >> 4) : (32u >> 4);
      const uint32_t b_kstep = p.b_mn ? (2048u >> 4) : (32u >> 4);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      for (int tile = pair; tile < total_tiles; tile += npairs, ++it) {
        int mt, nt, kb, kn;
        int half_unused; decode_tile(p, tile, mt, nt, kb, kn, half_unused);
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        mbar_wait(&tempty_bar[buf], acc_phase ^ 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_EMPTY);
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        for (int ki = 0; ki < kn; ++ki) {
          mbar_wait(&full_bar[stage], phase, abort_flag, p.status, FT_ERR_WAIT_FULL);
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + stage * L::STAGE_BYTES);
          const uint32_t sB = sA + L::A_BYTES;
          const uint64_t adesc = make_smem_desc(sA, a_lbo, 1024);
          const uint64_t bdesc = make_smem_desc(sB, b_lbo, 1024);
#pragma unroll
          for (int kk = 0; kk < GEMM_BK / 16; ++kk) {
            umma_ss_pair(tmem_d, adesc + kk * a_kstep, bdesc + kk * b_kstep, idesc,
                         (ki > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit_both(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        umma_commit_both(&tfull_bar[buf]);
      }
      // Tail: both accumulator buffers released, i.e. every epilogue warp of BOTH CTAs has sent
      // its (remote) arrival and it has landed here, before this CTA leaves.
      for (int i = 0; i < 2; ++i, ++it) {
        mbar_wait(&tempty_bar[it & 1], ((it >> 1) & 1) ^ 1, abort_flag, p.status,
                  FT_ERR_WAIT_TMEM_EMPTY);
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) ------------------------------
    const int q = warp & 3;
    const int chalf = (warp - 2) >> 2;
    uint8_t* my_epi = epi_base + (warp - 2) * L::EPI_BUF_BYTES;
    const uint32_t tempty0 = mapa_u32(smem_u32(&tempty_bar[0]), 0);
    int it = 0;
    int nstores = 0;
    for (int tile = pair; tile < total_tiles; tile += npairs, ++it) {
      int mt, nt, kb, kn;
      int half_unused; decode_tile(p, tile, mt, nt, kb, kn, half_unused);
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      mbar_wait(&tfull_bar[buf], acc_phase, abort_flag, p.status, FT_ERR_WAIT_TMEM_FULL);
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
      const int row0 = mt * 256 + static_cast<int>(rank) * 128 + q * 32;
      drain_tile(p, &tmD, taddr, row0, nt * BN, BN, chalf, my_epi, lane, nstores);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty0 + buf * 8);
    }
    if (lane == 0) tma_wait_group<0>();
    __syncwarp();
  }

  // Neither CTA may leave (or free its TMEM) while the other can still signal its barriers
  // or the issuing thread can still write its accumulators.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
  // Neither CTA leaves before BOTH have issued the pair-wide free: a CTA of another kernel that
  // got the first SM in between would otherwise have its fresh TMEM allocation there hit by
  // the second CTA's free.
  __syncwarp();
  cluster_sync_all();
}

#endif  // FT_BUILD_PAIR_GEMM

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
struct TmapKey {
  const void* base;
  uint64_t rows, cols, ld;
  uint32_t box_r, box_c, elt, swz;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_r == o.box_r &&
           box_c == o.box_c && elt == o.elt && swz == o.swz;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    auto mix = [&](uint64_t v) { h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2); };
    mix(k.rows); mix(k.cols); mix(k.ld); mix(k.box_r); mix(k.box_c); mix(k.elt); mix(k.swz);
    return h;
  }
};

static std::mutex g_tmap_mu;
static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> g_tmap_cache;

// Cached 2-D tensor map. A map only encodes address + geometry, so a cached entry stays valid
// for as long as the same geometry is asked for at the same address. The inner extent of the
// box in bytes has to EQUAL the swizzle span: with a shorter inner extent the rows of the box
// do not lie at the pitch of the inner extent in shared memory.
static int get_tmap_2d_swz(CUtensorMap* out, const void* base, int elt, uint64_t rows,
                           uint64_t cols, uint64_t ld, uint32_t box_r, uint32_t box_c,
                           CUtensorMapSwizzle swz) {
  TmapKey k{base, rows, cols, ld, box_r, box_c, static_cast<uint32_t>(elt),
            static_cast<uint32_t>(swz)};
  std::lock_guard<std::mutex> g(g_tmap_mu);
  auto it = g_tmap_cache.find(k);
  if (it != g_tmap_cache.end()) {
    *out = it->second;
    return 0;
  }
  CUtensorMap tm;
  int rc = make_tmap_2d(&tm, base, elt, rows, cols, ld, box_r, box_c, swz);
  if (rc) return rc;
  if (g_tmap_cache.size() > 65536) g_tmap_cache.clear();
  g_tmap_cache.emplace(k, tm);
  *out = tm;
  return 0;
}

// The 128-byte-swizzled map that every other kernel of the library uses.
int get_tmap_2d(CUtensorMap* out, const void* base, int elt, uint64_t rows, uint64_t cols,
                uint64_t ld, uint32_t box_r, uint32_t box_c) {
  return get_tmap_2d_swz(out, base, elt, rows, cols, ld, box_r, box_c,
                         CU_TENSOR_MAP_SWIZZLE_128B);
}

static int g_num_sms = 0;
static int num_sms() {
  if (!g_num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

template <int BN, int STAGES, int EPI = EPI_PLAIN>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmD,
                       const CUtensorMap& tmD2, const GemmParams& p, int max_ctas,
                       cudaStream_t stream) {
  using L = GemmSmem<BN, STAGES, EPI == EPI_SWIGLU_BWD ? 2 : 1>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BN, STAGES, EPI>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return -10;
    attr_set = true;
  }
  const int total = p.total_units;
  int grid = total < max_ctas ? total : max_ctas;
  if (grid < 1) grid = 1;
  gemm_bf16_kernel<BN, STAGES, EPI>
      <<<grid, GEMM_THREADS, L::TOTAL, stream>>>(tmA, tmB, tmD, tmD2, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

#ifdef FT_BUILD_PAIR_GEMM
static int launch_gemm_pair(const CUtensorMap& tmA, const CUtensorMap& tmB,
                            const CUtensorMap& tmD, const GemmParams& p, int max_ctas,
                            cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_bf16_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         PairSmem::TOTAL);
    if (e != cudaSuccess) return -10;
    attr_set = true;
  }
  const int total = p.m_tiles * p.n_tiles * p.splitk;
  int pairs = max_ctas / 2;
  if (pairs > total) pairs = total;
  if (pairs < 1) pairs = 1;
  gemm_pair_bf16_kernel<<<2 * pairs, GEMM_THREADS, PairSmem::TOTAL, stream>>>(tmA, tmB, tmD, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
#endif  // FT_BUILD_PAIR_GEMM

}  // namespace ft

// Tile selection, per shape class (what the rules below resolve to for the two model families at
// their benchmark token counts; TFLOP/s measured on a B200 at boost clock, cuBLAS in brackets):
//
//   shape (M x N x K)                 tile      split / tail              fwd    dgrad  wgrad
//   0.5B qkv      16384 x 1280 x 1024 128x256   tail: 48 tiles halved      975    999    819  (1135/1076/893)
//   0.5B attn_out 16384 x 1024 x 1024 128x256   tail: 68 tiles halved      932    932    780  ( 959/1015/818)
//   0.5B fc1      16384 x 8192 x 1024 128x256   -  (27.7 waves)           1370   1383   1316  (1498/1588/1627)
//   0.5B fc2      16384 x 1024 x 4096 128x256   tail: 68 tiles halved     1291   1329   1231  (1384/1329/1443)
//   0.5B lm_head  16384 x 73448 x 1024 128x256  -  (248 waves)            1224   1226   1164  (1117/1317/1556)
//   8B/TP2 qkv     8192 x 2304 x 4096 128x256   -                         1451   1452   1325  (1623/1438/1696)
//   8B/TP2 fc1     8192 x 16384 x 4096 128x256  -                         1473   1465   1219  (1404/1305/1545)
//   N <= 128 (test shapes only)       128x128   six stages
//   weight gradients whose M x N gives fewer tiles than SMs: split-K over the token dimension
//   (up to 16 ways, at least 8 k-steps per split), partial tiles summed by TMA reduce-add.
// The forward of fc1 and the dgrad of fc2 run the variants with the SwiGLU passes in their
// epilogues (ft_gemm_swiglu_bf16, ft_gemm_swiglu_bwd_bf16 below).
//
// D[M,N] (=|+=) alpha * A * B^T with bf16 operands.
//   a_mn == 0: A is stored [M][lda] (reduction index contiguous); a_mn == 1: A is stored
//   [K][lda] (row index contiguous). Same for B with N. out_dtype: 0 bf16, 1 fp32.
//   accumulate != 0 (fp32 only): D += result. splitk <= 0 picks a split automatically
//   (fp32 only); bn in {0 (auto), 128, 256}. All leading dimensions in elements; every base
//   pointer 16-byte aligned and every leading dimension a multiple of 8 (bf16) / 4 (fp32).
extern "C" int ft_gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K, int lda,
                            int ldb, int ldd, int a_mn, int b_mn, int out_dtype, int accumulate,
                            float alpha, int splitk, int bn, int max_ctas, int* status,
                            cudaStream_t stream) {
  using namespace ft;
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  if (out_dtype == 0 && accumulate) return -2;
  const int sms = num_sms();
  if (max_ctas <= 0 || max_ctas > sms) max_ctas = sms;
  const int k_iters = (K + GEMM_BK - 1) / GEMM_BK;
  // bn: 128 / 256 = one CTA per 128 x bn tile.
  if (bn != 128 && bn != 256) bn = (N <= 128) ? 128 : 256;
  constexpr bool pair = false;
  const int bm = GEMM_BM;
  const int m_tiles = (M + bm - 1) / bm;
  const int n_tiles = (N + bn - 1) / bn;
  if (out_dtype == 0) splitk = 1;
  if (splitk <= 0) {
    const int tiles = m_tiles * n_tiles;
    splitk = 1;
    const int units = pair ? max_ctas / 2 : max_ctas;
    if (tiles < units) {
      splitk = units / tiles;
      const int max_by_k = k_iters / 8 > 0 ? k_iters / 8 : 1;
      if (splitk > max_by_k) splitk = max_by_k;
      if (splitk > 16) splitk = 16;
    }
  }
  if (splitk > k_iters) splitk = k_iters;
  if (splitk < 1) splitk = 1;

  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.a_mn = a_mn ? 1 : 0; p.b_mn = b_mn ? 1 : 0;
  p.alpha = alpha;
  p.splitk = splitk;
  p.m_tiles = m_tiles; p.n_tiles = n_tiles; p.k_iters = k_iters;
  p.status = status;
  p.swiglu_F = 0;
  {
    // Tail of the schedule: when the last wave is at most half full, its tiles are cut in two
    // (128 x 128 halves on twice as many CTAs). Shapes of the 0.5B model at 16384 tokens: the
    // attention-output, FC2-forward and FC1-dgrad GEMMs have 512 tiles = 3.46 waves of 148, the
    // QKV forward 640 = 4.32; a half tile costs about 0.6 of a whole one.
    const int total = m_tiles * n_tiles * splitk;
    p.split_from = total;
    p.total_units = total;
    if (bn == 256 && splitk == 1 && max_ctas >= 2) {
      const int rem = total % max_ctas;
      if (rem > 0 && 2 * rem <= max_ctas) {
        p.split_from = total - rem;
        p.total_units = total + rem;
      }
    }
  }
  if (out_dtype == 0) p.out_mode = OUT_BF16;
  else p.out_mode = (accumulate || splitk > 1) ? OUT_F32_ADD : OUT_F32;
  if (out_dtype == 1 && !accumulate && splitk > 1) {
    if (cudaMemset2DAsync(D, static_cast<size_t>(ldd) * 4, 0, static_cast<size_t>(N) * 4, M,
                          stream) != cudaSuccess)
      return -3;
  }

  CUtensorMap tmA, tmB, tmD;
  int rc;
  if (!a_mn) rc = get_tmap_2d(&tmA, A, 2, M, K, lda, GEMM_BM, GEMM_BK);
  else       rc = get_tmap_2d(&tmA, A, 2, K, M, lda, GEMM_BK, 64);
  if (rc) return -4;
  if (!b_mn) rc = get_tmap_2d(&tmB, B, 2, N, K, ldb, 128, GEMM_BK);
  else       rc = get_tmap_2d(&tmB, B, 2, K, N, ldb, GEMM_BK, 64);
  if (rc) return -5;
  if (out_dtype == 0) rc = get_tmap_2d(&tmD, D, 2, M, N, ldd, 32, 64);
  else                rc = get_tmap_2d(&tmD, D, 4, M, N, ldd, 32, 32);
  if (rc) return -6;

  if (bn == 256) return launch_gemm<256, 4>(tmA, tmB, tmD, tmD, p, max_ctas, stream);
  return launch_gemm<128, 6>(tmA, tmB, tmD, tmD, p, max_ctas, stream);
}

// FC1 with the SwiGLU activation in the epilogue. A is [M][lda] activations, W is [2F][ldw] =
// [gate rows ; up rows] (both with the reduction index contiguous). Writes Y[M][2F] = alpha * A W^T
// (bf16, what the backward pass needs) and ACT[M][F] = silu(Y[:, :F]) * Y[:, F:] in one pass.
// F must be a multiple of 128 (a tile holds 128 gate columns and the matching 128 up columns).
extern "C" int ft_gemm_swiglu_bf16(const void* A, const void* W, void* Y, void* ACT, int M, int F,
                                   int K, int lda, int ldw, int ldy, int ldact, float alpha,
                                   int max_ctas, int* status, cudaStream_t stream) {
  using namespace ft;
  if (M <= 0 || F <= 0 || K <= 0) return -1;
  if (F % 128) return -2;
  const int sms = num_sms();
  if (max_ctas <= 0 || max_ctas > sms) max_ctas = sms;
  GemmParams p;
  p.M = M; p.N = 2 * F; p.K = K;
  p.a_mn = 0; p.b_mn = 0;
  p.out_mode = OUT_BF16;
  p.alpha = alpha;
  p.splitk = 1;
  p.m_tiles = (M + GEMM_BM - 1) / GEMM_BM;
  p.n_tiles = F / 128;
  p.k_iters = (K + GEMM_BK - 1) / GEMM_BK;
  p.status = status;
  p.swiglu_F = F;
  p.split_from = p.total_units = p.m_tiles * p.n_tiles;
  CUtensorMap tmA, tmB, tmY, tmAct;
  if (get_tmap_2d(&tmA, A, 2, M, K, lda, GEMM_BM, GEMM_BK)) return -4;
  if (get_tmap_2d(&tmB, W, 2, 2 * static_cast<uint64_t>(F), K, ldw, 128, GEMM_BK)) return -5;
  if (get_tmap_2d(&tmY, Y, 2, M, 2 * static_cast<uint64_t>(F), ldy, 32, 64)) return -6;
  if (get_tmap_2d(&tmAct, ACT, 2, M, F, ldact, 32, 64)) return -6;
  return launch_gemm<256, 4, EPI_SWIGLU_FWD>(tmA, tmB, tmY, tmAct, p, max_ctas, stream);
}

// FC2 dgrad with the SwiGLU backward in the epilogue: DY1[M][2F] = swiglu_bwd(alpha * DY W2, Y1),
// where DY is [M][ldy] (K = hidden size, reduction index contiguous), W2 is [K][ldw] with F
// contiguous columns, Y1 = [gate ; up] is the FC1 output of the forward pass. Bitwise equal to
// ft_gemm_bf16 (dgrad, bf16 out) followed by ft_swiglu_bwd. F must be a multiple of 64.
extern "C" int ft_gemm_swiglu_bwd_bf16(const void* DY, const void* W2, const void* Y1, void* DY1,
                                       int M, int F, int K, int lddy, int ldw, int ldy1,
                                       int lddy1, float alpha, int max_ctas, int* status,
                                       cudaStream_t stream) {
  using namespace ft;
  if (M <= 0 || F <= 0 || K <= 0) return -1;
  if (F % 64 || ldy1 % 8 || (reinterpret_cast<uintptr_t>(Y1) & 15)) return -2;
  const int sms = num_sms();
  if (max_ctas <= 0 || max_ctas > sms) max_ctas = sms;
  GemmParams p;
  p.M = M; p.N = F; p.K = K;
  p.a_mn = 0; p.b_mn = 1;
  p.out_mode = OUT_BF16;
  p.alpha = alpha;
  p.splitk = 1;
  p.m_tiles = (M + GEMM_BM - 1) / GEMM_BM;
  p.n_tiles = (F + 255) / 256;
  p.k_iters = (K + GEMM_BK - 1) / GEMM_BK;
  p.status = status;
  p.swiglu_F = F;
  const int total = p.m_tiles * p.n_tiles;
  p.split_from = p.total_units = total;
  const int rem = total % max_ctas;
  if (max_ctas >= 2 && rem > 0 && 2 * rem <= max_ctas) {
    p.split_from = total - rem;
    p.total_units = total + rem;
  }
  CUtensorMap tmA, tmB, tmD, tmY;
  if (get_tmap_2d(&tmA, DY, 2, M, K, lddy, GEMM_BM, GEMM_BK)) return -4;
  if (get_tmap_2d(&tmB, W2, 2, K, F, ldw, GEMM_BK, 64)) return -5;
  // boxes of 32 rows x 32 bf16 columns = 64-byte rows, 64-byte swizzle
  if (get_tmap_2d_swz(&tmD, DY1, 2, M, 2 * static_cast<uint64_t>(F), lddy1, 32, 32,
                      CU_TENSOR_MAP_SWIZZLE_64B))
    return -6;
  if (get_tmap_2d_swz(&tmY, Y1, 2, M, 2 * static_cast<uint64_t>(F), ldy1, 32, 32,
                      CU_TENSOR_MAP_SWIZZLE_64B))
    return -6;
  // three operand stages instead of four: the second staging buffer per epilogue warp needs 32 KB
  return launch_gemm<256, 3, EPI_SWIGLU_BWD>(tmA, tmB, tmD, tmY, p, max_ctas, stream);
}

extern "C" void ft_tmap_cache_clear() {
  std::lock_guard<std::mutex> g(ft::g_tmap_mu);
  ft::g_tmap_cache.clear();
}
