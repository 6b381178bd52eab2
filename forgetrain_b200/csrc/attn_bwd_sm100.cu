// Causal GQA FlashAttention backward for sm_100a (head_dim 64 or 128) on tcgen05 / TMEM / TMA.
//
// Three launches:
//   1. preprocess : delta[b,h,s] = sum_d out*dout, lse2 = lse * log2(e)
//   2. main       : one CTA per (kv tile of 128 rows, batch, kv group, chunk of query heads);
//                   it keeps K_j and V_j resident in shared memory and walks the query tiles
//                   i >= j of its heads. Per step, with everything transposed so that one
//                   thread owns one kv row:
//                     S^T = K Q^T, dP^T = V dO^T                      (tcgen05 -> TMEM)
//                     P^T = exp2(S^T*c - lse2), dS^T = P^T*(dP^T - delta)   (softmax warpgroup)
//                     dV += P^T dO, dK += dS^T Q, dQ = dS K           (tcgen05 -> TMEM)
//                   The same shared-memory tiles serve as K-major operands of the first two
//                   products and as MN-major operands of the last three, so nothing is
//                   transposed or copied. dQ tiles (every step) and dK/dV (once per CTA) are
//                   reduced into an fp32 accumulator laid out like the qkv buffer with vector
//                   reductions (red.global.add.v4.f32).
//   3. postprocess: accumulator * scale -> bf16 gradient of the interleaved qkv buffer.
//
// Replaces the reference's three-kernel Hopper backward
// (ops/attention/flash_attn_dsl/flash_bwd.py:243-3373).
#include "ptx.cuh"
#include "tma_host.h"

namespace ft {

int get_tmap_2d(CUtensorMap* out, const void* base, int elt, uint64_t rows, uint64_t cols,
                uint64_t ld, uint32_t box_r, uint32_t box_c);

constexpr int FAB_THREADS = 512;  // WG0: TMA + MMA, WG1/WG2: softmax halves, WG3: dQ / dK / dV drain
constexpr int FAB_BLK = 128;

struct FaBwdParams {
  int S, Hq, g, n_groups, batch, hpc;  // hpc: query heads per CTA
  int ld_acc;                          // row pitch (floats) of the fp32 accumulator
  float scale_log2;
  const float* lse2;   // [B][Hq][S]  lse * log2(e)
  const float* delta;  // [B][Hq][S]
  float* acc;          // [T][ld_acc] fp32, same column layout as qkv
  int* status;
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b),
               "f"(c), "f"(d)
               : "memory");
}

// QS: Q/dO stages, NP: P^T buffers in shared memory (0: P^T is kept in TMEM as packed bf16 and
// feeds the dV product as a TMEM operand), NDS: dS^T buffers, NST: (lse2, delta) buffers
template <int D, int QS, int NP, int NDS, int NST>
struct FaBwdSmem {
  static constexpr int TILE = FAB_BLK * D * 2;
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = TILE;
  static constexpr int QDO_OFF = 2 * TILE;                 // QS x (Q tile, dO tile)
  static constexpr int P_OFF = QDO_OFF + QS * 2 * TILE;    // NP x P^T (128 x 128 bf16)
  static constexpr int DS_OFF = P_OFF + NP * 32768;        // NDS x dS^T
  static constexpr int STAT_OFF = DS_OFF + NDS * 32768;    // NST x (lse2[128], delta[128]) fp32
  static constexpr int BAR_OFF = STAT_OFF + NST * 1024;
  static constexpr int TOTAL = BAR_OFF + 256;              // base must come 1024-byte aligned
};

template <int D, int QS, int NP, int NDS, int NST>
__global__ void __launch_bounds__(FAB_THREADS, 1)
fa_bwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_do,
              const FaBwdParams p) {
  using L = FaBwdSmem<D, QS, NP, NDS, NST>;
  constexpr bool ALIAS = (D == 128);  // dQ shares the TMEM columns of S^T
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
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
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
    mbar_init(dkv_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tm_qkv);
    prefetch_tmap(&tm_do);
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
  const uint32_t tm_dQ = ALIAS ? tmem_base : tmem_base + 256 + 2 * D;
  constexpr bool P_TMEM = (NP == 0);
  constexpr int NPB = P_TMEM ? 1 : NP;           // ring length of the P^T hand-over barriers
  const uint32_t tm_Pt = tmem_base + 448;        // 64 columns of packed bf16 (P_TMEM only)

  // step n -> (head, query tile)
  auto step_head = [&](int n) { return grp * p.g + hc * p.hpc + n / n_q; };
  auto step_qtile = [&](int n) { return j + n % n_q; };

  if (warp < 4) {
  reg_dealloc<88>();
  if (warp == 0) {
    if (lane == 0) {
      // ---------------- producer ----------------
      mbar_expect_tx(kv_full, 2 * L::TILE);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        tma_load_2d(smem + L::K_OFF + c * 16384, &tm_qkv, kv_full, k_col + c * 64,
                    row_base + j * FAB_BLK);
        tma_load_2d(smem + L::V_OFF + c * 16384, &tm_qkv, kv_full, v_col + c * 64,
                    row_base + j * FAB_BLK);
      }
      for (int n = 0; n < N; ++n) {
        const int s = n % QS;
        const int head = step_head(n), qt = step_qtile(n);
        const int q_col = (grp * (p.g + 2) + head % p.g) * D;
        mbar_wait(&qdo_empty[s], ((n / QS) & 1) ^ 1, abort_flag, p.status, FT_ERR_WAIT_EMPTY);
        mbar_expect_tx(&qdo_full[s], 2 * L::TILE + 1024);
        uint8_t* dst = smem + L::QDO_OFF + s * 2 * L::TILE;
        {
          const long soff = (static_cast<long>(b) * p.Hq + head) * p.S + qt * FAB_BLK;
          if (n >= NST)   // the (lse2, delta) slot is free once the softmax of step n-NST is done
            mbar_wait(&pds_ready[(n - NST) % NDS], ((n - NST) / NDS) & 1, abort_flag, p.status,
                      FT_ERR_WAIT_MISC);
          float* st = reinterpret_cast<float*>(smem + L::STAT_OFF + (n % NST) * 1024);
          bulk_load_1d(st, p.lse2 + soff, 512, &qdo_full[s]);
          bulk_load_1d(st + 128, p.delta + soff, 512, &qdo_full[s]);
        }
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          tma_load_2d(dst + c * 16384, &tm_qkv, &qdo_full[s], q_col + c * 64,
                      row_base + qt * FAB_BLK);
          tma_load_2d(dst + L::TILE + c * 16384, &tm_do, &qdo_full[s], head * D + c * 64,
                      row_base + qt * FAB_BLK);
        }
      }
      if (*abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer ----------------
      const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_dkv = make_idesc_bf16(128, D, 0, 1);
      const uint32_t idesc_dq = make_idesc_bf16(128, D, 1, 1);
      const uint32_t sK = smem_u32(smem + L::K_OFF), sV = smem_u32(smem + L::V_OFF);
      const uint32_t sQDO = smem_u32(smem + L::QDO_OFF);
      const uint32_t sP = smem_u32(smem + L::P_OFF), sDS = smem_u32(smem + L::DS_OFF);
      auto issue_sdp = [&](int n) {
        const int s = n % QS;
        mbar_wait(&qdo_full[s], (n / QS) & 1, abort_flag, p.status, FT_ERR_WAIT_FULL);
        tc_fence_after();
        const uint32_t q = sQDO + s * 2 * L::TILE, dO = q + L::TILE;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * 16384 + (kk % 4) * 32;
          umma_ss(tm_St, make_smem_desc(sK + off, 16, 1024), make_smem_desc(q + off, 16, 1024),
                  idesc_s, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * 16384 + (kk % 4) * 32;
          umma_ss(tm_dPt, make_smem_desc(sV + off, 16, 1024), make_smem_desc(dO + off, 16, 1024),
                  idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(sdp_full);
      };
      mbar_wait(kv_full, 0, abort_flag, p.status, FT_ERR_WAIT_FULL);
      issue_sdp(0);
      for (int n = 0; n < N; ++n) {
        const int s = n % QS;
        mbar_wait(&pds_ready[n % NDS], (n / NDS) & 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
        tc_fence_after();
        // With the single P^T buffer in TMEM, dV(n) goes first: it frees P^T before the softmax
        // of step n+1 (which needs S^T(n+1), issued right behind it) wants to write it.
        if (!ALIAS && !P_TMEM && n + 1 < N) issue_sdp(n + 1);
        const uint32_t q = sQDO + s * 2 * L::TILE, dO = q + L::TILE;
        const uint32_t dsT = sDS + (n % NDS) * 32768;
        if (P_TMEM) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)   // 16 bf16 of the reduction index = 8 TMEM columns
            umma_ts(tm_dV, tm_Pt + kk * 8, make_smem_desc(dO + kk * 2048, 16384, 1024), idesc_dkv,
                    (n > 0 || kk > 0) ? 1u : 0u);
        } else {
          const uint32_t pT = sP + (n % NPB) * 32768;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t aoff = (kk / 4) * 16384 + (kk % 4) * 32;
            umma_ss(tm_dV, make_smem_desc(pT + aoff, 16, 1024),
                    make_smem_desc(dO + kk * 2048, 16384, 1024), idesc_dkv,
                    (n > 0 || kk > 0) ? 1u : 0u);
          }
        }
        umma_commit(&p_free[n % NPB]);
        if (!ALIAS && P_TMEM && n + 1 < N) issue_sdp(n + 1);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t aoff = (kk / 4) * 16384 + (kk % 4) * 32;
          umma_ss(tm_dK, make_smem_desc(dsT + aoff, 16, 1024),
                  make_smem_desc(q + kk * 2048, 16384, 1024), idesc_dkv,
                  (n > 0 || kk > 0) ? 1u : 0u);
        }
        // Q_n / dO_n are last read by dK / dV: hand the stage back to the producer now
        umma_commit(&qdo_empty[s]);
        if (n > 0) {
          mbar_wait(dq_drained, (n - 1) & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_EMPTY);
          tc_fence_after();
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          umma_ss(tm_dQ, make_smem_desc(dsT + kk * 2048, 16384, 1024),
                  make_smem_desc(sK + kk * 2048, 16384, 1024), idesc_dq, kk > 0 ? 1u : 0u);
        }
        umma_commit(dq_full);
        umma_commit(&ds_free[n % NDS]);
        if (ALIAS && n + 1 < N) {
          mbar_wait(dq_drained, n & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_EMPTY);
          tc_fence_after();
          issue_sdp(n + 1);
        }
      }
      umma_commit(dkv_full);
    }
  }
  } else if (warp < 12) {
    reg_alloc<176>();
    // ---------------- two softmax warpgroups: thread owns kv row r and 64 of the 128 query
    // columns (warpgroup 1: columns 0-63, warpgroup 2: columns 64-127) ----------------
    const int half = (warp - 4) >> 2;
    const int r = (threadIdx.x - 128) & 127;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint64_t sl2x2 = pack_f32x2(p.scale_log2, p.scale_log2);
    for (int n = 0; n < N; ++n) {
      const int qt = step_qtile(n);
      const float* lse2 = reinterpret_cast<const float*>(smem + L::STAT_OFF + (n % NST) * 1024) + half * 64;
      const float* dlt = lse2 + 128;
      uint8_t* rowp = smem + L::P_OFF + (n % NPB) * 32768 + half * 16384 + r * 128;   // P^T row
      uint8_t* rowd = smem + L::DS_OFF + (n % NDS) * 32768 + half * 16384 + r * 128;  // dS^T row
      mbar_wait(&qdo_full[n % QS], (n / QS) & 1, abort_flag, p.status, FT_ERR_WAIT_FULL);
      mbar_wait(sdp_full, n & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_FULL);
      tc_fence_after();
      alignas(8) uint32_t s[64];
      alignas(8) uint32_t dp[64];
      tmem_ld32(tm_St + lane_off + half * 64, s);
      tmem_ld32(tm_St + lane_off + half * 64 + 32, s + 32);
      tmem_ld32(tm_dPt + lane_off + half * 64, dp);
      tmem_ld32(tm_dPt + lane_off + half * 64 + 32, dp + 32);
      tmem_ld_wait();
      // the buffers written below were last read by dV (P^T) and by dK / dQ (dS^T)
      mbar_wait(&p_free[n % NPB], ((n / NPB) & 1) ^ 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
      tc_fence_after();
      uint32_t pt[32];   // this thread's 64 P values as packed bf16 (P_TMEM)
      mbar_wait(&ds_free[n % NDS], ((n / NDS) & 1) ^ 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
      if (qt == j) {  // diagonal tile: query column < kv row is masked
#pragma unroll
        for (int k = 0; k < 64; ++k)
          if (half * 64 + k < r) s[k] = 0xff800000u;  // -inf -> p = 0
      }
      // Staged over the whole 64-column slice so that every stage is 32-64 independent
      // instructions (the per-element chain fma -> ex2 -> mul -> cvt is long and serial).
      uint64_t* s2 = reinterpret_cast<uint64_t*>(s);    // pairs of scores / probabilities
      uint64_t* d2 = reinterpret_cast<uint64_t*>(dp);   // pairs of dP / dS
#pragma unroll
      for (int i = 0; i < 16; ++i) {                    // t = s * scale - lse2 ; dd = dP - delta
        const float4 l4 = reinterpret_cast<const float4*>(lse2)[i];
        const float4 e4 = reinterpret_cast<const float4*>(dlt)[i];
        s2[2 * i] = fma_f32x2(s2[2 * i], sl2x2, pack_f32x2(-l4.x, -l4.y));
        s2[2 * i + 1] = fma_f32x2(s2[2 * i + 1], sl2x2, pack_f32x2(-l4.z, -l4.w));
        d2[2 * i] = add_f32x2(d2[2 * i], pack_f32x2(-e4.x, -e4.y));
        d2[2 * i + 1] = add_f32x2(d2[2 * i + 1], pack_f32x2(-e4.z, -e4.w));
      }
#pragma unroll
      for (int k = 0; k < 64; ++k) s[k] = __float_as_uint(fast_exp2(__uint_as_float(s[k])));
#pragma unroll
      for (int i = 0; i < 32; ++i) d2[i] = mul_f32x2(s2[i], d2[i]);   // dS = P * (dP - delta)
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint32_t pk[4], dk[4];
#pragma unroll
        for (int q2 = 0; q2 < 4; ++q2) {
          const int k = c * 8 + q2 * 2;
          pk[q2] = pack_bf16x2(__uint_as_float(s[k]), __uint_as_float(s[k + 1]));
          dk[q2] = pack_bf16x2(__uint_as_float(dp[k]), __uint_as_float(dp[k + 1]));
        }
        const int chunk = (c ^ (r & 7)) << 4;
        if (P_TMEM) {
#pragma unroll
          for (int q2 = 0; q2 < 4; ++q2) pt[c * 4 + q2] = pk[q2];
        } else {
          *reinterpret_cast<uint4*>(rowp + chunk) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
        *reinterpret_cast<uint4*>(rowd + chunk) = make_uint4(dk[0], dk[1], dk[2], dk[3]);
      }
      if (P_TMEM) {
        tmem_st32(tm_Pt + lane_off + half * 32, pt);
        tmem_st_wait();
      }
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(&pds_ready[n % NDS]);
    }
  } else {
    reg_dealloc<72>();
    // ---------------- drain warpgroup: dQ every step (thread r owns query row r), dK / dV at
    // the end (thread r owns kv row r) ----------------
    const int r = threadIdx.x - 384;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    for (int n = 0; n < N; ++n) {
      const int head = step_head(n), qt = step_qtile(n);
      const int q_col = (grp * (p.g + 2) + head % p.g) * D;
      float* acc_row = p.acc + static_cast<long>(row_base + qt * FAB_BLK + r) * p.ld_acc + q_col;
      mbar_wait(dq_full, n & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_FULL);
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(tm_dQ + lane_off + c * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int k = 0; k < 8; ++k)
          red_add_v4(acc_row + c * 32 + 4 * k, __uint_as_float(o[4 * k]),
                     __uint_as_float(o[4 * k + 1]), __uint_as_float(o[4 * k + 2]),
                     __uint_as_float(o[4 * k + 3]));
      }
      tc_fence_before();
      mbar_arrive(dq_drained);
    }
    mbar_wait(dkv_full, 0, abort_flag, p.status, FT_ERR_WAIT_TMEM_FULL);
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

// delta[b,h,s] = sum_d out*dout ; lse2 = lse*log2(e). One thread per 8 elements.
template <int D>
__global__ void fa_bwd_pre_kernel(const __nv_bfloat16* __restrict__ out,
                                  const __nv_bfloat16* __restrict__ dout,
                                  const float* __restrict__ lse, float* __restrict__ delta,
                                  float* __restrict__ lse2, long T, int S, int Hq, int ld_out,
                                  int ld_dout) {
  constexpr int TPH = D / 8;  // threads per (token, head)
  const long gid = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
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
    delta[idx] = acc;
    lse2[idx] = lse[idx] * 1.4426950408889634f;
  }
}

// dqkv[t][c] = bf16(acc[t][c] * (v column ? 1 : scale))
__global__ void fa_bwd_post_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dqkv,
                                   long T, int ncols, int ld_acc, int ld_dqkv, int g, int D,
                                   float scale) {
  const int vpr = ncols / 8;
  const long total = T * vpr;
  for (long idx = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long>(gridDim.x) * blockDim.x) {
    const long t = idx / vpr;
    const int c = (idx % vpr) * 8;
    const int in_grp = (c / D) % (g + 2);
    const float sc = (in_grp == g + 1) ? 1.f : scale;
    const float4 a = *reinterpret_cast<const float4*>(acc + t * ld_acc + c);
    const float4 b2 = *reinterpret_cast<const float4*>(acc + t * ld_acc + c + 4);
    uint4 o;
    o.x = pack_bf16x2(a.x * sc, a.y * sc);
    o.y = pack_bf16x2(a.z * sc, a.w * sc);
    o.z = pack_bf16x2(b2.x * sc, b2.y * sc);
    o.w = pack_bf16x2(b2.z * sc, b2.w * sc);
    *reinterpret_cast<uint4*>(dqkv + t * ld_dqkv + c) = o;
  }
}

template <int D, int QS, int NP, int NDS, int NST>
static int launch_fa_bwd(const CUtensorMap& tq, const CUtensorMap& tdo, const FaBwdParams& p,
                         cudaStream_t st) {
  using L = FaBwdSmem<D, QS, NP, NDS, NST>;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(fa_bwd_kernel<D, QS, NP, NDS, NST>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             L::TOTAL) != cudaSuccess)
      return -10;
    attr = true;
  }
  const int grid = (p.S / FAB_BLK) * p.batch * p.n_groups * (p.g / p.hpc);
  fa_bwd_kernel<D, QS, NP, NDS, NST><<<grid, FAB_THREADS, L::TOTAL, st>>>(tq, tdo, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace ft

// dout/out: [batch*S][ld] bf16 (head h at columns [h*D,(h+1)*D)); qkv / dqkv: interleaved
// layout; lse: [batch][Hq][S] fp32 from the forward. Scratch (caller-provided, fp32):
//   acc   [batch*S][ncols]  zero-filled by this call,  ncols = n_groups*(g+2)*D
//   delta [2][batch][Hq][S] (second half holds lse*log2(e))
// heads_per_cta <= 0 picks a value that keeps the grid well above the SM count.
extern "C" int ft_attn_bwd(const void* dout, const void* qkv, const void* out, const void* lse,
                           void* dqkv, void* acc, void* delta, int batch, int S, int n_groups,
                           int g, int D, int ld_qkv, int ld_out, int ld_dout, float scale,
                           int heads_per_cta, int* status, cudaStream_t st) {
  using namespace ft;
  if (S % FAB_BLK || (D != 64 && D != 128)) return -1;
  const long T = static_cast<long>(batch) * S;
  const int Hq = n_groups * g;
  const int ncols = n_groups * (g + 2) * D;
  if (heads_per_cta <= 0) {
    heads_per_cta = g;
    while (heads_per_cta > 1 &&
           static_cast<long>(S / FAB_BLK) * batch * n_groups * (g / heads_per_cta) < 148 * 6)
      heads_per_cta /= 2;
  }
  if (g % heads_per_cta) return -4;
  float* d_delta = static_cast<float*>(delta);
  float* d_lse2 = d_delta + static_cast<long>(batch) * Hq * S;
  if (cudaMemsetAsync(acc, 0, static_cast<size_t>(T) * ncols * 4, st) != cudaSuccess) return -5;
  {
    const long threads = T * Hq * (D / 8);
    const int blocks = static_cast<int>((threads + 255) / 256);
    if (D == 64)
      fa_bwd_pre_kernel<64><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)out,
                                                    (const __nv_bfloat16*)dout, (const float*)lse,
                                                    d_delta, d_lse2, T, S, Hq, ld_out, ld_dout);
    else
      fa_bwd_pre_kernel<128><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)out,
                                                     (const __nv_bfloat16*)dout, (const float*)lse,
                                                     d_delta, d_lse2, T, S, Hq, ld_out, ld_dout);
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
  int rc = (D == 64) ? launch_fa_bwd<64, 2, 2, 2, 2>(tq, tdo, p, st)
                     : launch_fa_bwd<128, 1, 1, 1, 1>(tq, tdo, p, st);
  if (rc) return rc;
  {
    const long total = T * (ncols / 8);
    long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    fa_bwd_post_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(
        (const float*)acc, (__nv_bfloat16*)dqkv, T, ncols, ncols, ld_qkv, g, D, scale);
    if (cudaGetLastError() != cudaSuccess) return -7;
  }
  return 0;
}
