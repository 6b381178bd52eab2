// Causal GQA FlashAttention backward, main kernel for head_dim 64, with the probabilities kept
// in TMEM. Everything is transposed so that one softmax thread owns one KV row (= one TMEM
// lane) and the two transposed products read their A operand straight from TMEM:
//
//   S^T  = K Q^T            (tcgen05, both operands from shared memory)        -> TMEM
//   P^T  = exp2(S^T c - lse2)                     softmax threads  -> TMEM (packed bf16)
//   dP^T = V dO^T           (into the columns S^T just left)                   -> TMEM
//   dS^T = P^T (dP^T - delta)                     softmax threads  -> TMEM (packed bf16)
//                                                          and -> shared memory (for dQ)
//   dV  += P^T dO           (A operand from TMEM)
//   dK  += dS^T Q           (A operand from TMEM)
//   dQ   = dS K             (A operand = the dS^T tile in shared memory, read MN-major)
//
// Against the variant that hands P and dS over through shared memory (attn_bwd_sm100.cu, still
// used at head_dim 128 where TMEM has no room) this takes 96 of 320 KB of shared-memory traffic
// per 128 x 128 step off the pipe that bounds the kernel, and the two TMEM-operand products
// run at the full tensor rate (an M=128, N=64 product with both operands in shared memory is
// bound by the A-operand fetch: 48 instead of 32 cycles per instruction, measured).
//
// TMEM columns: [0,128) S^T / dP^T, [128,192) dV, [192,256) dK, [256,320) dQ, [320,384) P^T,
// [384,448) dS^T. Work decomposition, producer, dQ / dK / dV drain and the fp32 accumulator are
// those of attn_bwd_sm100.cu.
#include "ptx.cuh"
#include "tma_host.h"

namespace ft {

struct FaBwdParams {
  int S, Hq, g, n_groups, batch, hpc;  // hpc: query heads per CTA
  int ld_acc;                          // row pitch (floats) of the fp32 accumulator
  float scale_log2;
  const float* lse2;   // [B][Hq][S]  -(lse * log2(e))
  const float* delta;  // [B][Hq][S]  -delta
  float* acc;          // [T][ld_acc] fp32, same column layout as qkv
  int* status;
};

constexpr int FABK_THREADS = 512;  // WG0: TMA + MMA, WG1/WG2: softmax halves, WG3: drain
constexpr int FABK_BLK = 128;
constexpr int FABK_D = 64;

__device__ __forceinline__ void kv_red_add_v2(float* addr, float a, float b) {
  asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(addr), "f"(a), "f"(b) : "memory");
}
__device__ __forceinline__ void kv_red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b),
               "f"(c), "f"(d)
               : "memory");
}

// QS: Q/dO stages (each with its (-lse2, -delta) rows), NDS: dS^T buffers in shared memory
template <int QS, int NDS>
struct FaBwdKvSmem {
  static constexpr int TILE = FABK_BLK * FABK_D * 2;        // 16 KB
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = TILE;
  static constexpr int QDO_OFF = 2 * TILE;                  // QS x (Q tile, dO tile)
  static constexpr int DS_OFF = QDO_OFF + QS * 2 * TILE;    // NDS x dS^T (128 kv x 128 q bf16)
  static constexpr int DQ_OFF = DS_OFF + NDS * 32768;       // dQ staging: 8 boxes of 32 x 32 fp32
  static constexpr int STAT_OFF = DQ_OFF + 32768;           // QS x (-lse2[128], -delta[128])
  static constexpr int BAR_OFF = STAT_OFF + QS * 1024;
  static constexpr int TOTAL = BAR_OFF + 512;               // base must come 1024-byte aligned
};

template <int QS, int NDS>
__global__ void __launch_bounds__(FABK_THREADS, 1)
fa_bwd_kv_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_do,
                 const __grid_constant__ CUtensorMap tm_acc, const FaBwdParams p) {
  using L = FaBwdKvSmem<QS, NDS>;
  constexpr int D = FABK_D;
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
  uint64_t* s_full = bars + 9;       // S^T of a step is in TMEM
  uint64_t* s_free = bars + 10;      // (count 256) ... and in registers: dP^T may overwrite it
  uint64_t* dp_full = bars + 11;     // dP^T of a step is in TMEM
  uint64_t* dp_free = bars + 12;     // (count 256) ... and in registers: the next S^T may come
  uint64_t* p_ready = bars + 13;     // (count 256) P^T of a step is stored in TMEM
  uint64_t* p_free = bars + 14;      // dV has read it
  uint64_t* pds_ready = bars + 15;   // 2 (count 256): dS^T of a step is stored (TMEM + smem)
  uint64_t* dst_free = bars + 17;    // dK has read dS^T from TMEM
  uint64_t* ds_free = bars + 18;     // 2: dQ has read the shared-memory dS^T buffer
  uint64_t* dq_full = bars + 20;     // 1
  uint64_t* dq_drained = bars + 21;  // 1 (count 128)
  uint64_t* dkv_full = bars + 22;    // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 24);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = warp_idx_uniform();
  const int lane = threadIdx.x & 31;

  // work decomposition: kv tile ascending = heavy first
  const int n_tiles = p.S / FABK_BLK;
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
    mbar_init(s_full, 1);
    mbar_init(s_free, 256);
    mbar_init(dp_full, 1);
    mbar_init(dp_free, 256);
    mbar_init(p_ready, 256);
    mbar_init(p_free, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&pds_ready[s], 256);
      mbar_init(&ds_free[s], 1);
    }
    mbar_init(dst_free, 1);
    mbar_init(dq_full, 1);
    mbar_init(dq_drained, 128);
    mbar_init(dkv_full, 1);
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
  const uint32_t tm_SdP = tmem_base;
  const uint32_t tm_dV = tmem_base + 128;
  const uint32_t tm_dK = tmem_base + 192;
  const uint32_t tm_dQ = tmem_base + 256;
  const uint32_t tm_Pt = tmem_base + 320;
  const uint32_t tm_dSt = tmem_base + 384;

  // step n -> (head, query tile)
  auto step_head = [&](int n) { return grp * p.g + hc * p.hpc + n / n_q; };
  auto step_qtile = [&](int n) { return j + n % n_q; };

  if (warp < 4) {
  reg_dealloc<88>();
  if (warp == 0) {
    // ---------------- producer: one load per lane (a thread that issues a TMA load is held
    // for several hundred cycles per instruction) ----------------
    if (lane < 4) {
      if (lane == 0) mbar_expect_tx(kv_full, 2 * L::TILE);
      if (lane == 0)
        tma_load_2d(smem + L::K_OFF, &tm_qkv, kv_full, k_col, row_base + j * FABK_BLK);
      else if (lane == 1)
        tma_load_2d(smem + L::V_OFF, &tm_qkv, kv_full, v_col, row_base + j * FABK_BLK);
      for (int n = 0; n < N; ++n) {
        const int s = n % QS;
        const int head = step_head(n), qt = step_qtile(n);
        const int q_col = (grp * (p.g + 2) + head % p.g) * D;
        mbar_wait_relaxed(&qdo_empty[s], ((n / QS) & 1) ^ 1, abort_flag, p.status, FT_ERR_WAIT_EMPTY);
        if (lane == 0) mbar_expect_tx(&qdo_full[s], 2 * L::TILE + 1024);
        uint8_t* dst = smem + L::QDO_OFF + s * 2 * L::TILE;
        if (lane == 0) {
          tma_load_2d(dst, &tm_qkv, &qdo_full[s], q_col, row_base + qt * FABK_BLK);
        } else if (lane == 1) {
          tma_load_2d(dst + L::TILE, &tm_do, &qdo_full[s], head * D, row_base + qt * FABK_BLK);
        } else {
          // the statistics rows live and die with the Q / dO stage: the stage is handed back
          // after dK of its step, i.e. after the softmax threads have finished with them
          const long soff = (static_cast<long>(b) * p.Hq + head) * p.S + qt * FABK_BLK;
          float* st = reinterpret_cast<float*>(smem + L::STAT_OFF + s * 1024);
          if (lane == 2)
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
    // ---------------- MMA issuer: the whole warp runs the loop and the waits, one elected
    // lane issues (descriptors and loop state stay warp-uniform) ----------------
    const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
    const uint32_t idesc_t = make_idesc_bf16(128, D, 0, 1);    // A from TMEM, B MN-major
    const uint32_t idesc_dq = make_idesc_bf16(128, D, 1, 1);   // dS (MN-major view of dS^T) x K
    const uint32_t sK = smem_u32(smem + L::K_OFF), sV = smem_u32(smem + L::V_OFF);
    const uint32_t sQDO = smem_u32(smem + L::QDO_OFF), sDS = smem_u32(smem + L::DS_OFF);
    // K-major operand, reduction step kk (16 elements): +(kk/4)*16384 + (kk%4)*32 bytes;
    // MN-major operand, reduction step kk (16 rows of 128 B): + kk*2048 bytes.
    const uint32_t kK = smem_desc_lo(sK, 16), vK = smem_desc_lo(sV, 16);
    const uint32_t kMN = smem_desc_lo(sK, 16384);
    const uint32_t qK0 = smem_desc_lo(sQDO, 16), qMN0 = smem_desc_lo(sQDO, 16384);
    const uint32_t dsMN0 = smem_desc_lo(sDS, 16384);
    constexpr uint32_t STG = (2 * L::TILE) >> 4, TL = L::TILE >> 4, BUF = 32768 >> 4;
#define FT_KOFF(kk) ((((kk) / 4) * 16384 + ((kk) % 4) * 32) >> 4)
#define FT_MNOFF(kk) (((kk) * 2048) >> 4)
    auto wait_qdo = [&](int n) {
      mbar_wait(&qdo_full[n % QS], (n / QS) & 1, abort_flag, p.status, FT_ERR_WAIT_FULL);
      tc_fence_after();
    };
    auto issue_s = [&](int n) {            // S^T = K Q^T
      const uint32_t qK = qK0 + (n % QS) * STG;
      umma_ss_lo<0>(tm_SdP, kK, qK, idesc_s);
#pragma unroll
      for (int kk = 1; kk < D / 16; ++kk)
        umma_ss_lo<1>(tm_SdP, kK + FT_KOFF(kk), qK + FT_KOFF(kk), idesc_s);
      umma_commit(s_full);
    };
    auto issue_dp = [&](int n) {           // dP^T = V dO^T, into the columns of S^T
      const uint32_t doK = qK0 + (n % QS) * STG + TL;
      umma_ss_lo<0>(tm_SdP, vK, doK, idesc_s);
#pragma unroll
      for (int kk = 1; kk < D / 16; ++kk)
        umma_ss_lo<1>(tm_SdP, vK + FT_KOFF(kk), doK + FT_KOFF(kk), idesc_s);
      umma_commit(dp_full);
    };
    auto issue_dv = [&](int n) {           // dV += P^T dO, A from TMEM
      const uint32_t doMN = qMN0 + (n % QS) * STG + TL;
      umma_ts_lo_dyn(tm_dV, tm_Pt, doMN, idesc_t, n > 0 ? 1u : 0u);
#pragma unroll
      for (int kk = 1; kk < 8; ++kk)
        umma_ts_lo<1>(tm_dV, tm_Pt + kk * 8, doMN + FT_MNOFF(kk), idesc_t);
      umma_commit(p_free);
    };
    auto issue_dk = [&](int n) {           // dK += dS^T Q, A from TMEM
      const uint32_t qMN = qMN0 + (n % QS) * STG;
      umma_ts_lo_dyn(tm_dK, tm_dSt, qMN, idesc_t, n > 0 ? 1u : 0u);
#pragma unroll
      for (int kk = 1; kk < 8; ++kk)
        umma_ts_lo<1>(tm_dK, tm_dSt + kk * 8, qMN + FT_MNOFF(kk), idesc_t);
      umma_commit(dst_free);
      // Q_n / dO_n are last read by dK / dV: hand the stage back to the producer now
      umma_commit(&qdo_empty[n % QS]);
    };
    auto issue_dq = [&](int n) {           // dQ = dS K
      const uint32_t dsMN = dsMN0 + (n % NDS) * BUF;
      umma_ss_lo<0>(tm_dQ, dsMN, kMN, idesc_dq);
#pragma unroll
      for (int kk = 1; kk < 8; ++kk)
        umma_ss_lo<1>(tm_dQ, dsMN + FT_MNOFF(kk), kMN + FT_MNOFF(kk), idesc_dq);
      umma_commit(dq_full);
      umma_commit(&ds_free[n % NDS]);
    };
    mbar_wait(kv_full, 0, abort_flag, p.status, FT_ERR_WAIT_FULL);
    wait_qdo(0);
    if (elect_one_sync()) issue_s(0);
    __syncwarp();
    for (int n = 0; n < N; ++n) {
      // dP^T of this step as soon as the softmax threads hold S^T in registers
      mbar_wait(s_free, n & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_EMPTY);
      tc_fence_after();
      if (elect_one_sync()) issue_dp(n);
      __syncwarp();
      mbar_wait(p_ready, n & 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
      tc_fence_after();
      if (elect_one_sync()) issue_dv(n);
      __syncwarp();
      // S^T of the next step as soon as dP^T of this one is in registers: the next softmax
      // then starts without waiting for the tensor pipe
      if (n + 1 < N) {
        mbar_wait(dp_free, n & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_EMPTY);
        wait_qdo(n + 1);
        if (elect_one_sync()) issue_s(n + 1);
        __syncwarp();
      }
      mbar_wait(&pds_ready[n % NDS], (n / NDS) & 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
      tc_fence_after();
      if (elect_one_sync()) issue_dk(n);
      __syncwarp();
      if (n > 0) {
        mbar_wait(dq_drained, (n - 1) & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_EMPTY);
        tc_fence_after();
      }
      if (elect_one_sync()) issue_dq(n);
      __syncwarp();
    }
#undef FT_KOFF
#undef FT_MNOFF
    if (elect_one_sync()) umma_commit(dkv_full);
    __syncwarp();
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
      const float4* nl4 = reinterpret_cast<const float4*>(smem + L::STAT_OFF + (n % QS) * 1024) + half * 16;
      const float4* nd4 = nl4 + 32;
      uint8_t* rowd = smem + L::DS_OFF + (n % NDS) * 32768 + half * 16384 + r * 128;  // dS^T row
      mbar_wait(&qdo_full[n % QS], (n / QS) & 1, abort_flag, p.status, FT_ERR_WAIT_FULL);
      mbar_wait(s_full, n & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_FULL);
      tc_fence_after();
      alignas(8) uint32_t s[64];
      tmem_ld32(tm_SdP + lane_off + half * 64, s);
      tmem_ld32(tm_SdP + lane_off + half * 64 + 32, s + 32);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(s_free);
      if (qt == j) {  // diagonal tile: query column < kv row is masked
#pragma unroll
        for (int k = 0; k < 64; ++k)
          if (half * 64 + k < r) s[k] = 0xff800000u;  // -inf -> p = 0
      }
      uint64_t* s2 = reinterpret_cast<uint64_t*>(s);    // pairs of scores, then probabilities
      uint32_t w[32];                                   // packed bf16 row piece (P^T, then dS^T)
      // P^T = exp2(S^T * scale - lse2): scale, exponential and packing as one interleaved stream
      // (a warp can issue an `ex2` only every ~16 cycles; the rest goes out in the gaps)
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const float4 l = nl4[c];                         // -lse2 of four query columns
        const uint64_t t0 = fma_f32x2(s2[2 * c], sl2x2, pack_f32x2(l.x, l.y));
        const uint64_t t1 = fma_f32x2(s2[2 * c + 1], sl2x2, pack_f32x2(l.z, l.w));
        float a0, a1, a2, a3;
        unpack_f32x2(t0, a0, a1);
        unpack_f32x2(t1, a2, a3);
        a0 = fast_exp2(a0); a1 = fast_exp2(a1); a2 = fast_exp2(a2); a3 = fast_exp2(a3);
        s2[2 * c] = pack_f32x2(a0, a1);
        s2[2 * c + 1] = pack_f32x2(a2, a3);
        w[2 * c] = pack_bf16x2(a0, a1);
        w[2 * c + 1] = pack_bf16x2(a2, a3);
      }
      if (n > 0) {   // dV of the previous step has read P^T
        mbar_wait(p_free, (n - 1) & 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
        tc_fence_after();
      }
      tmem_st32(tm_Pt + lane_off + half * 32, w);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(p_ready);
      // dP^T arrived in the columns S^T left
      mbar_wait(dp_full, n & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_FULL);
      tc_fence_after();
      alignas(8) uint32_t dp[64];
      tmem_ld32(tm_SdP + lane_off + half * 64, dp);
      tmem_ld32(tm_SdP + lane_off + half * 64 + 32, dp + 32);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(dp_free);
      uint64_t* d2 = reinterpret_cast<uint64_t*>(dp);
#pragma unroll
      for (int c = 0; c < 16; ++c) {                     // dS^T = P^T * (dP^T - delta)
        const float4 dl = nd4[c];                        // -delta of four query columns
        const uint64_t x0 = mul_f32x2(s2[2 * c], add_f32x2(d2[2 * c], pack_f32x2(dl.x, dl.y)));
        const uint64_t x1 = mul_f32x2(s2[2 * c + 1], add_f32x2(d2[2 * c + 1], pack_f32x2(dl.z, dl.w)));
        float a0, a1, a2, a3;
        unpack_f32x2(x0, a0, a1);
        unpack_f32x2(x1, a2, a3);
        w[2 * c] = pack_bf16x2(a0, a1);
        w[2 * c + 1] = pack_bf16x2(a2, a3);
      }
      // dK of the previous step has read dS^T from TMEM; dQ of step n-NDS the smem buffer
      if (n > 0) {
        mbar_wait(dst_free, (n - 1) & 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
        tc_fence_after();
      }
      mbar_wait(&ds_free[n % NDS], ((n / NDS) & 1) ^ 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
      tmem_st32(tm_dSt + lane_off + half * 32, w);
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4*>(rowd + ((c ^ (r & 7)) << 4)) =
            make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
      tmem_st_wait();
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(&pds_ready[n % NDS]);
    }
  } else {
    reg_dealloc<72>();
    // ---------------- drain warpgroup: dQ every step (thread r owns query row r), dK / dV at
    // the end (thread r owns kv row r). The dQ tile leaves through TMA reduce-adds: each warp
    // stages its 32 rows as two swizzled 32 x 32 fp32 boxes and one lane sends them off, so the
    // fp32 accumulation in L2 is done by the copy engine in whole 128-byte lines. (Per-thread
    // `red.global` instructions for the same bytes kept the load / store pipe of the SM so busy
    // that the softmax warps' own shared-memory traffic stalled behind them: the kernel ran
    // 1.45x slower.) ----------------
    const int r = threadIdx.x - 384;
    const int q4 = warp & 3;
    const uint32_t lane_off = static_cast<uint32_t>(q4 * 32) << 16;
    uint8_t* stage = smem + L::DQ_OFF + q4 * 8192;           // this warp's two 4 KB boxes
    for (int n = 0; n < N; ++n) {
      const int head = step_head(n), qt = step_qtile(n);
      const int q_col = (grp * (p.g + 2) + head % p.g) * D;
      mbar_wait_relaxed(dq_full, n & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_FULL);
      tc_fence_after();
      uint32_t o[64];
      tmem_ld32(tm_dQ + lane_off, o);
      tmem_ld32(tm_dQ + lane_off + 32, o + 32);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(dq_drained);                 // the accumulator is in registers: dQ of the next step may start
      if (n > 0) {                             // the previous step's boxes have been read
        if (lane == 0) tma_wait_group_read<0>();
        __syncwarp();
      }
#pragma unroll
      for (int hb = 0; hb < 2; ++hb)
#pragma unroll
        for (int c = 0; c < 8; ++c)
          *reinterpret_cast<uint4*>(stage + hb * 4096 + lane * 128 + ((c ^ (lane & 7)) << 4)) =
              make_uint4(o[hb * 32 + 4 * c], o[hb * 32 + 4 * c + 1], o[hb * 32 + 4 * c + 2],
                         o[hb * 32 + 4 * c + 3]);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        const int y = row_base + qt * FABK_BLK + q4 * 32;
        tma_reduce_add_2d(&tm_acc, stage, q_col, y);
        tma_reduce_add_2d(&tm_acc, stage + 4096, q_col + 32, y);
        tma_commit_group();
      }
    }
    if (lane == 0) tma_wait_group<0>();
    __syncwarp();
    mbar_wait_relaxed(dkv_full, 0, abort_flag, p.status, FT_ERR_WAIT_TMEM_FULL, 256);
    tc_fence_after();
    float* acc_row = p.acc + static_cast<long>(row_base + j * FABK_BLK + r) * p.ld_acc;
#pragma unroll 1
    for (int c = 0; c < D / 32; ++c) {
      uint32_t o[32];
      tmem_ld32(tm_dV + lane_off + c * 32, o);
      tmem_ld_wait();
#pragma unroll
      for (int k = 0; k < 8; ++k)
        kv_red_add_v4(acc_row + v_col + c * 32 + 4 * k, __uint_as_float(o[4 * k]),
                      __uint_as_float(o[4 * k + 1]), __uint_as_float(o[4 * k + 2]),
                      __uint_as_float(o[4 * k + 3]));
      tmem_ld32(tm_dK + lane_off + c * 32, o);
      tmem_ld_wait();
#pragma unroll
      for (int k = 0; k < 8; ++k)
        kv_red_add_v4(acc_row + k_col + c * 32 + 4 * k, __uint_as_float(o[4 * k]),
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

// Launch of the TMEM-operand main kernel (head_dim 64). Same contract as the main kernel of
// attn_bwd_sm100.cu; `lse2` and `delta` hold the NEGATED statistics; `tacc` is a 32 x 32 fp32
// box map over the accumulator.
int launch_fa_bwd_kv64(const CUtensorMap& tq, const CUtensorMap& tdo, const CUtensorMap& tacc,
                       int S, int Hq, int g,
                       int n_groups, int batch, int hpc, int ld_acc, float scale_log2,
                       const float* neg_lse2, const float* neg_delta, float* acc, int* status,
                       cudaStream_t st) {
  using L = FaBwdKvSmem<3, 1>;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(fa_bwd_kv_kernel<3, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             L::TOTAL) != cudaSuccess)
      return -10;
    attr = true;
  }
  FaBwdParams p;
  p.S = S; p.Hq = Hq; p.g = g; p.n_groups = n_groups; p.batch = batch; p.hpc = hpc;
  p.ld_acc = ld_acc;
  p.scale_log2 = scale_log2;
  p.lse2 = neg_lse2; p.delta = neg_delta; p.acc = acc;
  p.status = status;
  const int grid = (S / FABK_BLK) * batch * n_groups * (g / hpc);
  fa_bwd_kv_kernel<3, 1><<<grid, FABK_THREADS, L::TOTAL, st>>>(tq, tdo, tacc, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace ft
