// Causal GQA FlashAttention backward for sm_100a (head_dim 64 or 128) on tcgen05 / TMEM / TMA.
//
// Three launches:
//   1. preprocess : delta[b,h,s] = sum_d out*dout, lse2 = lse * log2(e)
//   2. main       : one CTA per (kv tile of 128 rows, batch, kv group, chunk of query heads);
//                   it keeps K_j and V_j resident in shared memory and walks the query tiles
//                   i >= j of its heads. Per step, with one softmax thread per QUERY row (its
//                   lse2 and delta are then two scalars, not a vector re-read per element):
//                     S = Q K^T, dP = dO V^T                          (tcgen05 -> TMEM)
//                     P = exp2(S*c - lse2), dS = P*(dP - delta)       (softmax warpgroups)
//                     dV += P^T dO, dK += dS^T Q, dQ = dS K           (tcgen05 -> TMEM)
//                   P and dS are stored once, as [query][kv] tiles; the transposed products
//                   read them as MN-major A operands and dQ reads dS as a K-major one, and the
//                   Q / dO / K tiles likewise serve as K-major operands of the first two
//                   products and as MN-major B operands of the last three, so nothing is
//                   transposed or copied. dQ tiles (every step) and dK/dV (once per CTA) are
//                   reduced into an fp32 accumulator laid out like the qkv buffer with vector
//                   reductions (red.global.add.v4.f32).
//   3. postprocess: accumulator * scale -> bf16 gradient of the interleaved qkv buffer.
//
// Replaces the reference's three-kernel Hopper backward
// (ops/attention/flash_attn_dsl/flash_bwd.py:243-3373).
#include <stdlib.h>

#include "ptx.cuh"
#include "tma_host.h"

namespace ft {

int get_tmap_2d(CUtensorMap* out, const void* base, int elt, uint64_t rows, uint64_t cols,
                uint64_t ld, uint32_t box_r, uint32_t box_c);
// main kernel for head_dim 64 (P^T / dS^T kept in TMEM), attn_bwd_kv_sm100.cu
int launch_fa_bwd_kv64(const CUtensorMap& tq, const CUtensorMap& tdo, const CUtensorMap& tacc,
                       int S, int Hq, int g,
                       int n_groups, int batch, int hpc, int ld_acc, float scale_log2,
                       const float* neg_lse2, const float* neg_delta, float* acc, int* status,
                       cudaStream_t st);
int launch_fa_bwd_kv128(const CUtensorMap& tkv, const CUtensorMap& tq, const CUtensorMap& tdo,
                        const CUtensorMap& tacc, int S, int Hq, int g, int n_groups, int batch,
                        int hpc, int ld_acc, float scale_log2, const float* neg_lse2,
                        const float* neg_delta, float* acc, int* status, cudaStream_t st);

constexpr int FAB_THREADS = 512;  // WG0: TMA + MMA, WG1/WG2: softmax halves, WG3: dQ / dK / dV drain
constexpr int FAB_BLK = 128;

struct FaBwdParams {
  int S, Hq, g, n_groups, batch, hpc;  // hpc: query heads per CTA
  int ld_acc;                          // row pitch (floats) of the fp32 accumulator
  float scale_log2;
  const float* lse2;   // [B][Hq][S]  -(lse * log2(e))
  const float* delta;  // [B][Hq][S]  -delta
  float* acc;          // [T][ld_acc] fp32, same column layout as qkv
  int* status;
};

__device__ __forceinline__ void red_add_v2(float* addr, float a, float b) {
  asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(addr), "f"(a), "f"(b) : "memory");
}
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b),
               "f"(c), "f"(d)
               : "memory");
}

// QS: Q/dO stages, NP: P buffers in shared memory, NDS: dS buffers, NST: (lse2, delta) buffers
template <int D, int QS, int NP, int NDS, int NST>
struct FaBwdSmem {
  static constexpr int TILE = FAB_BLK * D * 2;
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = TILE;
  static constexpr int QDO_OFF = 2 * TILE;                 // QS x (Q tile, dO tile)
  static constexpr int P_OFF = QDO_OFF + QS * 2 * TILE;    // NP x P^T (128 x 128 bf16)
  static constexpr int DS_OFF = P_OFF + NP * 32768;        // NDS x dS^T
  static constexpr int DQ_OFF = DS_OFF + NDS * 32768;      // dQ staging: 8 boxes of 32 x 32 fp32
  static constexpr int STAT_OFF = DQ_OFF + 32768;          // NST x (lse2[128], delta[128]) fp32
  static constexpr int BAR_OFF = STAT_OFF + NST * 1024;
  static constexpr int TOTAL = BAR_OFF + 256;              // base must come 1024-byte aligned
};

template <int D, int QS, int NP, int NDS, int NST>
__global__ void __launch_bounds__(FAB_THREADS, 1)
fa_bwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_do,
              const __grid_constant__ CUtensorMap tm_acc, const FaBwdParams p) {
  using L = FaBwdSmem<D, QS, NP, NDS, NST>;
  // head_dim 128 fills all 512 TMEM columns with S, dP, dV and dK, so dQ has to share the
  // columns of dP. The step is then split: S of step n+1 is issued as soon as S of step n is in
  // registers and the softmax warpgroups exponentiate it (and dV starts) while dQ of step n is
  // still being drained; only dP of step n+1 waits for the drain.
  constexpr bool ALIAS = (D == 128);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023u) {  // swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, FT_ERR_WAIT_MISC);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* kv_full = bars;          // 1
  uint64_t* qdo_full = bars + 1;     // 4
  uint64_t* qdo_empty = bars + 5;    // 4
  uint64_t* sdp_full = bars + 9;     // 1
  uint64_t* pds_ready = bars + 10;   // 2 (count 256): P^T and dS^T of a step are written
  uint64_t* ds_free = bars + 12;     // 2: dS^T buffer consumed by dK and dQ
  uint64_t* p_free = bars + 14;      // 2: P^T buffer consumed by dV
  uint64_t* dq_full = bars + 16;     // 1
  uint64_t* dq_drained = bars + 17;  // 1 (count 128)
  uint64_t* dkv_full = bars + 18;    // 1
  uint64_t* sdp_free = bars + 19;    // 1 (count 256): S (and dP) of a step are in registers
  uint64_t* dp_full = bars + 20;     // 1: dP of a step is in TMEM (head_dim 128 only)
  uint64_t* p_ready = bars + 21;     // 2 (count 256): P of a step is written (head_dim 128 only)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 24);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = warp_idx_uniform();
  const int lane = threadIdx.x & 31;

  // work decomposition: kv tile ascending = heavy first
  const int n_tiles = p.S / FAB_BLK;
  const int chunks = p.g / p.hpc;
  int bid = blockIdx.x;
  const int hc = bid % chunks; bid /= chunks;
  const int grp = bid % p.n_groups; bid /= p.n_groups;
  const int b = bid % p.batch; bid /= p.batch;
  const int j = bid;  // kv tile
  const int k_col = (grp * (p.g + 2) + p.g) * D;
  const int v_col = k_col + D;
  const int row_base = b * p.S;
  const int n_q = n_tiles - j;     // query tiles j .. n_tiles-1
  const int N = p.hpc * n_q;       // steps of this CTA

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 4; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&qdo_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&pds_ready[s], 256);
      mbar_init(&ds_free[s], 1);
      mbar_init(&p_free[s], 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(dq_full, 1);
    mbar_init(dq_drained, 128);
    mbar_init(dp_full, 1);
    mbar_init(&p_ready[0], 256);
    mbar_init(&p_ready[1], 256);
    mbar_init(dkv_full, 1);
    mbar_init(sdp_free, 256);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tm_qkv);
    prefetch_tmap(&tm_do);
    prefetch_tmap(&tm_acc);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_St = tmem_base;
  const uint32_t tm_dPt = tmem_base + 128;
  const uint32_t tm_dV = tmem_base + 256;
  const uint32_t tm_dK = tmem_base + 256 + D;
  const uint32_t tm_dQ = ALIAS ? tm_dPt : tmem_base + 256 + 2 * D;
  static_assert(NP >= 1 && NDS >= 1, "P and dS are handed over through shared memory");
  constexpr int NPB = NP;                        // ring length of the P hand-over barriers

  // step n -> (head, query tile)
  auto step_head = [&](int n) { return grp * p.g + hc * p.hpc + n / n_q; };
  auto step_qtile = [&](int n) { return j + n % n_q; };

  if (warp < 4) {
  reg_dealloc<88>();
  if (warp == 0) {
    // ---------------- producer ----------------
    // A thread that issues a TMA load is held for several hundred cycles per instruction, so
    // the loads of a step (Q and dO boxes, lse2 and delta rows) are spread over lanes: one
    // instruction issues them all.
    constexpr int NBOX = D / 64;            // 64-column boxes per tile
    constexpr int NL = 2 * NBOX + 2;
    if (lane < NL) {
      if (lane == 0) mbar_expect_tx(kv_full, 2 * L::TILE);
      if (lane < 2 * NBOX) {
        const int c = lane % NBOX;
        if (lane < NBOX)
          tma_load_2d(smem + L::K_OFF + c * 16384, &tm_qkv, kv_full, k_col + c * 64,
                      row_base + j * FAB_BLK);
        else
          tma_load_2d(smem + L::V_OFF + c * 16384, &tm_qkv, kv_full, v_col + c * 64,
                      row_base + j * FAB_BLK);
      }
      for (int n = 0; n < N; ++n) {
        const int s = n % QS;
        const int head = step_head(n), qt = step_qtile(n);
        const int q_col = (grp * (p.g + 2) + head % p.g) * D;
        mbar_wait_relaxed(&qdo_empty[s], ((n / QS) & 1) ^ 1, abort_flag, p.status, FT_ERR_WAIT_EMPTY);
        if (lane == 0) mbar_expect_tx(&qdo_full[s], 2 * L::TILE + 1024);
        uint8_t* dst = smem + L::QDO_OFF + s * 2 * L::TILE;
        if (lane < NBOX) {
          tma_load_2d(dst + lane * 16384, &tm_qkv, &qdo_full[s], q_col + lane * 64,
                      row_base + qt * FAB_BLK);
        } else if (lane < 2 * NBOX) {
          const int c = lane - NBOX;
          tma_load_2d(dst + L::TILE + c * 16384, &tm_do, &qdo_full[s], head * D + c * 64,
                      row_base + qt * FAB_BLK);
        } else {
          const long soff = (static_cast<long>(b) * p.Hq + head) * p.S + qt * FAB_BLK;
          if (n >= NST)   // the (lse2, delta) slot is free once the softmax of step n-NST is done
            mbar_wait_relaxed(&pds_ready[(n - NST) % NDS], ((n - NST) / NDS) & 1, abort_flag,
                              p.status, FT_ERR_WAIT_MISC);
          float* st = reinterpret_cast<float*>(smem + L::STAT_OFF + (n % NST) * 1024);
          if (lane == 2 * NBOX)
            bulk_load_1d(st, p.lse2 + soff, 512, &qdo_full[s]);
          else
            bulk_load_1d(st + 128, p.delta + soff, 512, &qdo_full[s]);
        }
      }
      if (lane == 0 && *abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    {
      // ---------------- MMA issuer: the whole warp runs the loop and the waits, one elected
      // lane issues (descriptors and loop state stay warp-uniform) ----------------
      const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_dkv = make_idesc_bf16(128, D, 1, 1);   // P^T / dS^T: MN-major A
      const uint32_t idesc_dq = make_idesc_bf16(128, D, 0, 1);    // dS: K-major A
      const uint32_t sK = smem_u32(smem + L::K_OFF), sV = smem_u32(smem + L::V_OFF);
      const uint32_t sQDO = smem_u32(smem + L::QDO_OFF);
      const uint32_t sP = smem_u32(smem + L::P_OFF), sDS = smem_u32(smem + L::DS_OFF);
      // Descriptor low words of the resident tiles; per-step tiles add their stage offset.
      // K-major operand, reduction step kk (16 elements): +(kk/4)*16384 + (kk%4)*32 bytes;
      // MN-major operand, reduction step kk (16 rows of 128 B): + kk*2048 bytes.
      const uint32_t kK = smem_desc_lo(sK, 16), vK = smem_desc_lo(sV, 16);
      const uint32_t kMN = smem_desc_lo(sK, 16384);
      const uint32_t qK0 = smem_desc_lo(sQDO, 16), qMN0 = smem_desc_lo(sQDO, 16384);
      const uint32_t pMN0 = smem_desc_lo(sP, 16384);
      const uint32_t dsK0 = smem_desc_lo(sDS, 16), dsMN0 = smem_desc_lo(sDS, 16384);
      constexpr uint32_t STG = (2 * L::TILE) >> 4, TL = L::TILE >> 4, BUF = 32768 >> 4;
#define FT_KOFF(kk) ((((kk) / 4) * 16384 + ((kk) % 4) * 32) >> 4)
#define FT_MNOFF(kk) (((kk) * 2048) >> 4)
      auto wait_qdo = [&](int n) {
        mbar_wait(&qdo_full[n % QS], (n / QS) & 1, abort_flag, p.status, FT_ERR_WAIT_FULL);
        tc_fence_after();
      };
      auto issue_s = [&](int n) {
        const int s = n % QS;
        const uint32_t qK = qK0 + s * STG;
        umma_ss_lo<0>(tm_St, qK, kK, idesc_s);
#pragma unroll
        for (int kk = 1; kk < D / 16; ++kk)
          umma_ss_lo<1>(tm_St, qK + FT_KOFF(kk), kK + FT_KOFF(kk), idesc_s);
        if (ALIAS) umma_commit(sdp_full);
      };
      auto issue_dp = [&](int n) {   // after issue_s(n): Q/dO of the step are known to be loaded
        const uint32_t doK = qK0 + (n % QS) * STG + TL;
        umma_ss_lo<0>(tm_dPt, doK, vK, idesc_s);
#pragma unroll
        for (int kk = 1; kk < D / 16; ++kk)
          umma_ss_lo<1>(tm_dPt, doK + FT_KOFF(kk), vK + FT_KOFF(kk), idesc_s);
        umma_commit(ALIAS ? dp_full : sdp_full);
      };
      auto issue_dv = [&](int n) {
        const uint32_t doMN = qMN0 + (n % QS) * STG + TL;
        const uint32_t pMN = pMN0 + (n % NPB) * BUF;
        umma_ss_lo_dyn(tm_dV, pMN, doMN, idesc_dkv, n > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 1; kk < 8; ++kk)
          umma_ss_lo<1>(tm_dV, pMN + FT_MNOFF(kk), doMN + FT_MNOFF(kk), idesc_dkv);
        umma_commit(&p_free[n % NPB]);
      };
      auto issue_dk = [&](int n) {
        const uint32_t qMN = qMN0 + (n % QS) * STG;
        const uint32_t dsMN = dsMN0 + (n % NDS) * BUF;
        umma_ss_lo_dyn(tm_dK, dsMN, qMN, idesc_dkv, n > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 1; kk < 8; ++kk)
          umma_ss_lo<1>(tm_dK, dsMN + FT_MNOFF(kk), qMN + FT_MNOFF(kk), idesc_dkv);
        // Q_n / dO_n are last read by dK / dV: hand the stage back to the producer now
        umma_commit(&qdo_empty[n % QS]);
      };
      auto issue_dq = [&](int n) {
        const uint32_t dsK = dsK0 + (n % NDS) * BUF;
        umma_ss_lo<0>(tm_dQ, dsK, kMN, idesc_dq);
#pragma unroll
        for (int kk = 1; kk < 8; ++kk)
          umma_ss_lo<1>(tm_dQ, dsK + FT_KOFF(kk), kMN + FT_MNOFF(kk), idesc_dq);
        umma_commit(dq_full);
        umma_commit(&ds_free[n % NDS]);
      };
      mbar_wait(kv_full, 0, abort_flag, p.status, FT_ERR_WAIT_FULL);
      wait_qdo(0);
      if (elect_one_sync()) {
        issue_s(0);
        issue_dp(0);
      }
      __syncwarp();
      for (int n = 0; n < N; ++n) {
        if (!ALIAS) {
          // S / dP of step n+1 go to the tensor pipe as soon as the softmax warpgroups hold
          // step n's scores in registers, i.e. while they are still computing P / dS of step
          // n: the next softmax then starts without waiting for these products.
          if (n + 1 < N) {
            mbar_wait(sdp_free, n & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_EMPTY);
            wait_qdo(n + 1);
            if (elect_one_sync()) {
              issue_s(n + 1);
              issue_dp(n + 1);
            }
            __syncwarp();
          }
          mbar_wait(&pds_ready[n % NDS], (n / NDS) & 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
          tc_fence_after();
          if (elect_one_sync()) {
            issue_dv(n);
            issue_dk(n);
          }
          __syncwarp();
          if (n > 0) {
            mbar_wait(dq_drained, (n - 1) & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_EMPTY);
            tc_fence_after();
          }
          if (elect_one_sync()) {
            issue_dq(n);
          }
          __syncwarp();
        } else {
          mbar_wait(&p_ready[n % NPB], (n / NPB) & 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
          tc_fence_after();
          if (elect_one_sync()) issue_dv(n);
          __syncwarp();
          mbar_wait(&pds_ready[n % NDS], (n / NDS) & 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
          tc_fence_after();
          if (elect_one_sync()) {
            issue_dk(n);
            issue_dq(n);   // into the columns of dP(n), which the softmax has read by now
          }
          __syncwarp();
          if (n + 1 < N) {
            mbar_wait(sdp_free, n & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_EMPTY);
            wait_qdo(n + 1);
            if (elect_one_sync()) issue_s(n + 1);
            __syncwarp();
            mbar_wait(dq_drained, n & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_EMPTY);
            tc_fence_after();
            if (elect_one_sync()) issue_dp(n + 1);
            __syncwarp();
          }
        }
      }
#undef FT_KOFF
#undef FT_MNOFF
      if (elect_one_sync()) umma_commit(dkv_full);
      __syncwarp();
    }
  }
  } else if (warp < 12) {
    reg_alloc<176>();
    // ---------------- two softmax warpgroups: thread owns query row r and 64 of the 128 kv
    // columns (warpgroup 1: columns 0-63, warpgroup 2: columns 64-127) ----------------
    const int half = (warp - 4) >> 2;
    const int r = (threadIdx.x - 128) & 127;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint64_t sl2x2 = pack_f32x2(p.scale_log2, p.scale_log2);
    for (int n = 0; n < N; ++n) {
      const int qt = step_qtile(n);
      const float* stat = reinterpret_cast<const float*>(smem + L::STAT_OFF + (n % NST) * 1024);
      uint8_t* rowp = smem + L::P_OFF + (n % NPB) * 32768 + half * 16384 + r * 128;   // P row
      uint8_t* rowd = smem + L::DS_OFF + (n % NDS) * 32768 + half * 16384 + r * 128;  // dS row
      mbar_wait(&qdo_full[n % QS], (n / QS) & 1, abort_flag, p.status, FT_ERR_WAIT_FULL);
      const float nl = stat[r], nd = stat[128 + r];   // the statistics are stored negated
      const uint64_t nl2 = pack_f32x2(nl, nl), nd2 = pack_f32x2(nd, nd);
      mbar_wait(sdp_full, n & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_FULL);
      tc_fence_after();
      alignas(8) uint32_t s[64];
      alignas(8) uint32_t dp[64];
      tmem_ld32(tm_St + lane_off + half * 64, s);
      tmem_ld32(tm_St + lane_off + half * 64 + 32, s + 32);
      if (!ALIAS) {
        tmem_ld32(tm_dPt + lane_off + half * 64, dp);
        tmem_ld32(tm_dPt + lane_off + half * 64 + 32, dp + 32);
      }
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(sdp_free);
      if (qt == j) {  // diagonal tile: kv column > query row is masked
#pragma unroll
        for (int k = 0; k < 64; ++k)
          if (half * 64 + k > r) s[k] = 0xff800000u;  // -inf -> p = 0
      }
      uint64_t* s2 = reinterpret_cast<uint64_t*>(s);    // pairs of scores / probabilities
      uint64_t* d2 = reinterpret_cast<uint64_t*>(dp);   // pairs of dP / dS
      if (ALIAS) {
        // P goes out first (dV can start); dP of this step arrives once dQ of the previous
        // step has left the columns the two share.
#pragma unroll
        for (int i = 0; i < 32; ++i) s2[i] = fma_f32x2(s2[i], sl2x2, nl2);   // t = s * scale - lse2
#pragma unroll
        for (int k = 0; k < 64; ++k) s[k] = __float_as_uint(fast_exp2(__uint_as_float(s[k])));
        mbar_wait(&p_free[n % NPB], ((n / NPB) & 1) ^ 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint32_t pk[4];
#pragma unroll
          for (int q2 = 0; q2 < 4; ++q2) {
            const int k = c * 8 + q2 * 2;
            pk[q2] = pack_bf16x2(__uint_as_float(s[k]), __uint_as_float(s[k + 1]));
          }
          *reinterpret_cast<uint4*>(rowp + ((c ^ (r & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
        tc_fence_before();
        fence_proxy_async_smem();
        mbar_arrive(&p_ready[n % NPB]);
        mbar_wait(dp_full, n & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_FULL);
        tc_fence_after();
        tmem_ld32(tm_dPt + lane_off + half * 64, dp);
        tmem_ld32(tm_dPt + lane_off + half * 64 + 32, dp + 32);
        tmem_ld_wait();
        mbar_wait(&ds_free[n % NDS], ((n / NDS) & 1) ^ 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint32_t dk[4];
#pragma unroll
          for (int q2 = 0; q2 < 4; ++q2) {
            const int i = c * 4 + q2;
            const uint64_t ds = mul_f32x2(s2[i], add_f32x2(d2[i], nd2));   // dS = P * (dP - delta)
            float a, b2;
            unpack_f32x2(ds, a, b2);
            dk[q2] = pack_bf16x2(a, b2);
          }
          *reinterpret_cast<uint4*>(rowd + ((c ^ (r & 7)) << 4)) = make_uint4(dk[0], dk[1], dk[2], dk[3]);
        }
      } else {
        // the buffers written below were last read by dV (P) and by dK / dQ (dS) of an earlier
        // step: long done in the steady state
        mbar_wait(&p_free[n % NPB], ((n / NPB) & 1) ^ 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
        mbar_wait(&ds_free[n % NDS], ((n / NDS) & 1) ^ 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
        // One interleaved stream over 8 chunks of 8 columns: a warp can issue an `ex2` only
        // every ~16 cycles, so scale, exponential, dS = P * (dP - delta), the two bf16 packings
        // and the two shared-memory stores go out in the gaps instead of in stages of their own.
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint32_t pk[4], dk[4];
#pragma unroll
          for (int q2 = 0; q2 < 4; ++q2) {
            const int i = c * 4 + q2;
            const uint64_t t = fma_f32x2(s2[i], sl2x2, nl2);               // s * scale - lse2
            float e0, e1;
            unpack_f32x2(t, e0, e1);
            e0 = fast_exp2(e0);
            e1 = fast_exp2(e1);
            const uint64_t ds = mul_f32x2(pack_f32x2(e0, e1), add_f32x2(d2[i], nd2));
            float a, b2;
            unpack_f32x2(ds, a, b2);
            pk[q2] = pack_bf16x2(e0, e1);
            dk[q2] = pack_bf16x2(a, b2);
          }
          const int chunk = (c ^ (r & 7)) << 4;
          *reinterpret_cast<uint4*>(rowp + chunk) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          *reinterpret_cast<uint4*>(rowd + chunk) = make_uint4(dk[0], dk[1], dk[2], dk[3]);
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(&pds_ready[n % NDS]);
    }
  } else {
    reg_dealloc<72>();
    // ---------------- drain warpgroup: dQ every step (thread r owns query row r), dK / dV at
    // the end (thread r owns kv row r) ----------------
    // The dQ tile leaves through TMA reduce-adds: each warp stages 32 rows x 64 columns as two
    // swizzled 32 x 32 fp32 boxes and one lane sends them off, so the fp32 accumulation in L2 is
    // done by the copy engine in whole 128-byte lines (per-thread `red.global` instructions for
    // the same bytes keep the SM's load / store pipe so busy that the softmax warps' own
    // shared-memory traffic stalls behind them).
    const int r = threadIdx.x - 384;
    const int q4 = warp & 3;
    const uint32_t lane_off = static_cast<uint32_t>(q4 * 32) << 16;
    uint8_t* stage = smem + L::DQ_OFF + q4 * 8192;           // this warp's two 4 KB boxes
    int nsent = 0;
    for (int n = 0; n < N; ++n) {
      const int head = step_head(n), qt = step_qtile(n);
      const int q_col = (grp * (p.g + 2) + head % p.g) * D;
      mbar_wait_relaxed(dq_full, n & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_FULL);
      tc_fence_after();
      const int y = row_base + qt * FAB_BLK + q4 * 32;
#pragma unroll 1
      for (int c = 0; c < D / 64; ++c) {
        uint32_t o[64];
        tmem_ld32(tm_dQ + lane_off + c * 64, o);
        tmem_ld32(tm_dQ + lane_off + c * 64 + 32, o + 32);
        tmem_ld_wait();
        if (c == D / 64 - 1) {     // the accumulator is in registers: the columns are free again
          tc_fence_before();
          mbar_arrive(dq_drained);
        }
        if (nsent > 0) {           // the boxes sent last have been read
          if (lane == 0) tma_wait_group_read<0>();
          __syncwarp();
        }
#pragma unroll
        for (int hb = 0; hb < 2; ++hb)
#pragma unroll
          for (int k = 0; k < 8; ++k)
            *reinterpret_cast<uint4*>(stage + hb * 4096 + lane * 128 + ((k ^ (lane & 7)) << 4)) =
                make_uint4(o[hb * 32 + 4 * k], o[hb * 32 + 4 * k + 1], o[hb * 32 + 4 * k + 2],
                           o[hb * 32 + 4 * k + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_reduce_add_2d(&tm_acc, stage, q_col + c * 64, y);
          tma_reduce_add_2d(&tm_acc, stage + 4096, q_col + c * 64 + 32, y);
          tma_commit_group();
        }
        ++nsent;
      }
    }
    if (lane == 0) tma_wait_group<0>();
    __syncwarp();
    mbar_wait_relaxed(dkv_full, 0, abort_flag, p.status, FT_ERR_WAIT_TMEM_FULL, 256);
    tc_fence_after();
    float* acc_row = p.acc + static_cast<long>(row_base + j * FAB_BLK + r) * p.ld_acc;
#pragma unroll 1
    for (int c = 0; c < D / 32; ++c) {
      uint32_t o[32];
      tmem_ld32(tm_dV + lane_off + c * 32, o);
      tmem_ld_wait();
#pragma unroll
      for (int k = 0; k < 8; ++k)
        red_add_v4(acc_row + v_col + c * 32 + 4 * k, __uint_as_float(o[4 * k]),
                   __uint_as_float(o[4 * k + 1]), __uint_as_float(o[4 * k + 2]),
                   __uint_as_float(o[4 * k + 3]));
      tmem_ld32(tm_dK + lane_off + c * 32, o);
      tmem_ld_wait();
#pragma unroll
      for (int k = 0; k < 8; ++k)
        red_add_v4(acc_row + k_col + c * 32 + 4 * k, __uint_as_float(o[4 * k]),
                   __uint_as_float(o[4 * k + 1]), __uint_as_float(o[4 * k + 2]),
                   __uint_as_float(o[4 * k + 3]));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b,h,s] = -sum_d out*dout ; lse2 = -lse*log2(e). One thread per 8 elements. The same
// pass zeroes the fp32 accumulator (`acc4`: n_acc4 float4) that the main kernel reduces into, so
// no separate fill runs and the stores ride along with this kernel's loads.
template <int D>
__global__ void fa_bwd_pre_kernel(const __nv_bfloat16* __restrict__ out,
                                  const __nv_bfloat16* __restrict__ dout,
                                  const float* __restrict__ lse, float* __restrict__ delta,
                                  float* __restrict__ lse2, long T, int S, int Hq, int ld_out,
                                  int ld_dout, float4* __restrict__ acc4, long n_acc4) {
  constexpr int TPH = D / 8;  // threads per (token, head)
  const long gid = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  {
    const long nthreads = static_cast<long>(gridDim.x) * blockDim.x;
    for (long k = gid; k < n_acc4; k += nthreads) acc4[k] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const long pair = gid / TPH;
  const int sub = gid % TPH;
  const bool live = pair < T * Hq;
  const long t = live ? pair / Hq : 0;
  const int h = live ? pair % Hq : 0;
  float acc = 0.f;
  if (live) {
    const uint4 a = *reinterpret_cast<const uint4*>(out + t * ld_out + h * D + sub * 8);
    const uint4 c = *reinterpret_cast<const uint4*>(dout + t * ld_dout + h * D + sub * 8);
    const uint32_t av[4] = {a.x, a.y, a.z, a.w}, cv[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) acc += bf16_lo(av[i]) * bf16_lo(cv[i]) + bf16_hi(av[i]) * bf16_hi(cv[i]);
  }
#pragma unroll
  for (int o = TPH / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (live && sub == 0) {
    const long bidx = t / S, s = t % S;
    const long idx = (bidx * Hq + h) * S + s;
    delta[idx] = -acc;     // both statistics are stored negated: the main kernels only add them
    lse2[idx] = -lse[idx] * 1.4426950408889634f;
  }
}

// dqkv[t][c] = bf16(acc[t][c] * (v column ? 1 : scale)), and, when a rotary table is given, the
// transposed rotation of the q and k heads (the backward of RoPE) in the same pass: one thread
// owns 8 columns of a head's first half and the matching 8 of its second half.
__global__ void fa_bwd_post_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dqkv,
                                   long T, int ncols, int ld_acc, int ld_dqkv, int g, int D,
                                   float scale, const float* __restrict__ cos_t,
                                   const float* __restrict__ sin_t,
                                   const int* __restrict__ position_ids, int S) {
  const int half = D / 2;
  const int vph = half / 8;                 // threads per head
  const int heads = ncols / D;
  const long total = T * heads * vph;
  for (long idx = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long>(gridDim.x) * blockDim.x) {
    const int v = idx % vph;
    const long r1 = idx / vph;
    const int hs = r1 % heads;
    const long t = r1 / heads;
    const bool is_v = (hs % (g + 2)) == g + 1;
    const float sc = is_v ? 1.f : scale;
    const int c0 = hs * D + v * 8;
    const float* a = acc + t * ld_acc + c0;
    float x1[8], x2[8];
    *reinterpret_cast<float4*>(x1) = *reinterpret_cast<const float4*>(a);
    *reinterpret_cast<float4*>(x1 + 4) = *reinterpret_cast<const float4*>(a + 4);
    *reinterpret_cast<float4*>(x2) = *reinterpret_cast<const float4*>(a + half);
    *reinterpret_cast<float4*>(x2 + 4) = *reinterpret_cast<const float4*>(a + half + 4);
#pragma unroll
    for (int k = 0; k < 8; ++k) { x1[k] *= sc; x2[k] *= sc; }
    if (cos_t != nullptr && !is_v) {
      const int pos = position_ids ? position_ids[t] : static_cast<int>(t % S);
      float c[8], sn[8];
      const float4* c4 = reinterpret_cast<const float4*>(cos_t + static_cast<long>(pos) * half + v * 8);
      const float4* s4 = reinterpret_cast<const float4*>(sin_t + static_cast<long>(pos) * half + v * 8);
      *reinterpret_cast<float4*>(c) = c4[0];
      *reinterpret_cast<float4*>(c + 4) = c4[1];
      *reinterpret_cast<float4*>(sn) = s4[0];
      *reinterpret_cast<float4*>(sn + 4) = s4[1];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float o1 = x1[k] * c[k] + x2[k] * sn[k];
        const float o2 = x2[k] * c[k] - x1[k] * sn[k];
        x1[k] = o1;
        x2[k] = o2;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(x1[0], x1[1]); o.y = pack_bf16x2(x1[2], x1[3]);
    o.z = pack_bf16x2(x1[4], x1[5]); o.w = pack_bf16x2(x1[6], x1[7]);
    *reinterpret_cast<uint4*>(dqkv + t * ld_dqkv + c0) = o;
    o.x = pack_bf16x2(x2[0], x2[1]); o.y = pack_bf16x2(x2[2], x2[3]);
    o.z = pack_bf16x2(x2[4], x2[5]); o.w = pack_bf16x2(x2[6], x2[7]);
    *reinterpret_cast<uint4*>(dqkv + t * ld_dqkv + c0 + half) = o;
  }
}

template <int D, int QS, int NP, int NDS, int NST>
static int launch_fa_bwd(const CUtensorMap& tq, const CUtensorMap& tdo, const CUtensorMap& tacc,
                         const FaBwdParams& p, cudaStream_t st) {
  using L = FaBwdSmem<D, QS, NP, NDS, NST>;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(fa_bwd_kernel<D, QS, NP, NDS, NST>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             L::TOTAL) != cudaSuccess)
      return -10;
    attr = true;
  }
  const int grid = (p.S / FAB_BLK) * p.batch * p.n_groups * (p.g / p.hpc);
  fa_bwd_kernel<D, QS, NP, NDS, NST><<<grid, FAB_THREADS, L::TOTAL, st>>>(tq, tdo, tacc, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace ft

// dout/out: [batch*S][ld] bf16 (head h at columns [h*D,(h+1)*D)); qkv / dqkv: interleaved
// layout; lse: [batch][Hq][S] fp32 from the forward. Scratch (caller-provided, fp32):
//   acc   [batch*S][ncols]  zero-filled by this call,  ncols = n_groups*(g+2)*D
//   delta [2][batch][Hq][S] (second half holds lse*log2(e))
// heads_per_cta <= 0 picks the largest value that keeps the grid at three CTAs per SM or more
// (measured optimum: longer CTAs amortise the K/V load and the dK/dV drain, but the causal
// triangle needs a few waves to balance).
// cos_t / sin_t ([positions][D/2] fp32, may be NULL) and position_ids ([batch*S] int32 or NULL =
// position inside the sequence): when given, the gradient of the q and k heads leaves with the
// backward of the rotary embedding already applied (no separate pass over the buffer).
extern "C" int ft_attn_bwd(const void* dout, const void* qkv, const void* out, const void* lse,
                           void* dqkv, void* acc, void* delta, int batch, int S, int n_groups,
                           int g, int D, int ld_qkv, int ld_out, int ld_dout, float scale,
                           int heads_per_cta, const void* cos_t, const void* sin_t,
                           const void* position_ids, int* status, cudaStream_t st) {
  using namespace ft;
  if (S % FAB_BLK || (D != 64 && D != 128)) return -1;
  const long T = static_cast<long>(batch) * S;
  const int Hq = n_groups * g;
  const int ncols = n_groups * (g + 2) * D;
  if (heads_per_cta <= 0) {
    heads_per_cta = g;
    while (heads_per_cta > 1 &&
           static_cast<long>(S / FAB_BLK) * batch * n_groups * (g / heads_per_cta) < 148 * 3)
      heads_per_cta /= 2;
  }
  if (g % heads_per_cta) return -4;
  float* d_delta = static_cast<float*>(delta);
  float* d_lse2 = d_delta + static_cast<long>(batch) * Hq * S;
  if (ncols % 4 || (reinterpret_cast<uintptr_t>(acc) & 15)) return -5;
  const long n_acc4 = T * ncols / 4;   // the accumulator is zeroed by the preprocess kernel
  {
    const long threads = T * Hq * (D / 8);
    const int blocks = static_cast<int>((threads + 255) / 256);
    if (D == 64)
      fa_bwd_pre_kernel<64><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)out,
                                                    (const __nv_bfloat16*)dout, (const float*)lse,
                                                    d_delta, d_lse2, T, S, Hq, ld_out, ld_dout,
                                                    static_cast<float4*>(acc), n_acc4);
    else
      fa_bwd_pre_kernel<128><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)out,
                                                     (const __nv_bfloat16*)dout, (const float*)lse,
                                                     d_delta, d_lse2, T, S, Hq, ld_out, ld_dout,
                                                     static_cast<float4*>(acc), n_acc4);
    if (cudaGetLastError() != cudaSuccess) return -6;
  }
  CUtensorMap tq, tdo;
  if (get_tmap_2d(&tq, qkv, 2, T, ncols, ld_qkv, FAB_BLK, 64)) return -2;
  if (get_tmap_2d(&tdo, dout, 2, T, static_cast<uint64_t>(Hq) * D, ld_dout, FAB_BLK, 64)) return -3;
  FaBwdParams p;
  p.S = S; p.Hq = Hq; p.g = g; p.n_groups = n_groups; p.batch = batch; p.hpc = heads_per_cta;
  p.ld_acc = ncols;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.lse2 = d_lse2; p.delta = d_delta; p.acc = static_cast<float*>(acc);
  p.status = status;
  CUtensorMap tacc;   // 32 x 32 fp32 boxes over the accumulator (dQ leaves through TMA reduce-adds)
  if (get_tmap_2d(&tacc, acc, 4, T, ncols, ncols, 32, 32)) return -8;
#ifndef FT_FAB_SMEM_P64
  int rc;
  if (D == 64) {
    rc = launch_fa_bwd_kv64(tq, tdo, tacc, S, Hq, g, n_groups, batch, heads_per_cta, ncols,
                            p.scale_log2, d_lse2, d_delta, p.acc, status, st);
  } else {
#ifndef FT_FAB_SMEM_P128
    // head_dim 128: the TMEM-operand kernel walks the query rows in tiles of 64
    CUtensorMap tq64, tdo64;
    if (get_tmap_2d(&tq64, qkv, 2, T, ncols, ld_qkv, 64, 64)) return -2;
    if (get_tmap_2d(&tdo64, dout, 2, T, static_cast<uint64_t>(Hq) * D, ld_dout, 64, 64)) return -3;
    rc = launch_fa_bwd_kv128(tq, tq64, tdo64, tacc, S, Hq, g, n_groups, batch, heads_per_cta,
                             ncols, p.scale_log2, d_lse2, d_delta, p.acc, status, st);
#else   // the shared-memory hand-over kernel (comparison builds)
    rc = launch_fa_bwd<128, 1, 1, 1, 1>(tq, tdo, tacc, p, st);
#endif
  }
#else   // head_dim 64 on the shared-memory hand-over kernel as well (comparison builds)
  int rc = (D == 64) ? launch_fa_bwd<64, 3, 1, 1, 2>(tq, tdo, tacc, p, st)
                     : launch_fa_bwd<128, 1, 1, 1, 1>(tq, tdo, tacc, p, st);
#endif
  if (rc) return rc;
  {
    const long total = T * (ncols / 16);
    long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    fa_bwd_post_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(
        (const float*)acc, (__nv_bfloat16*)dqkv, T, ncols, ncols, ld_qkv, g, D, scale,
        (const float*)cos_t, (const float*)sin_t, (const int*)position_ids, S);
    if (cudaGetLastError() != cudaSuccess) return -7;
  }
  return 0;
}
