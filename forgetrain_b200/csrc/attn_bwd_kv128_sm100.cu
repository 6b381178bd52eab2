// Causal GQA FlashAttention backward, main kernel for head_dim 128, with the probabilities kept
// in TMEM: the head_dim 64 kernel of attn_bwd_kv_sm100.cu restated for 128-wide heads. A CTA owns
// one 128-row KV tile; to fit K, V (64 KB) and a three-deep ring of Q / dO tiles in shared memory
// it walks the query rows in tiles of 64. One softmax thread owns one KV row (= one TMEM lane):
//
//   S^T  = K Q^T            [128 kv x 64 q]   both operands from shared memory      -> TMEM
//   P^T  = exp2(S^T c - lse2)                  softmax threads -> TMEM (packed bf16)
//   dP^T = V dO^T           [128 kv x 64 q]                                         -> TMEM
//   dS^T = P^T (dP^T - delta)                  softmax threads -> TMEM (packed bf16)
//                                                        and -> shared memory (for dQ)
//   dV  += P^T dO           [128 kv x 128 d]   A operand from TMEM, K = 64
//   dK  += dS^T Q           [128 kv x 128 d]   A operand from TMEM, K = 64
//   dQ^T = K^T dS^T         [128 d  x 64 q]    K tile read MN-major, dS^T tile from shared memory
//
// dQ is produced TRANSPOSED (lane = head-dim index) so that every product keeps M = 128; the
// drain warpgroup transposes it on its way into the staging boxes of the TMA reduce-adds.
// TMEM columns: [0,64) S^T, [64,128) dP^T, [128,256) dV, [256,384) dK, [384,448) dQ^T,
// [448,480) P^T, [480,512) dS^T. Work decomposition, statistics (negated lse2 / delta), the fp32
// accumulator and the conversion pass are those of attn_bwd_sm100.cu.
#include "ptx.cuh"
#include "tma_host.h"

namespace ft {

struct FaBwd128Params {
  int S, Hq, g, n_groups, batch, hpc;  // hpc: query heads per CTA
  int ld_acc;                          // row pitch (floats) of the fp32 accumulator
  float scale_log2;
  const float* lse2;   // [B][Hq][S]  -(lse * log2(e))
  const float* delta;  // [B][Hq][S]  -delta
  float* acc;          // [T][ld_acc] fp32, same column layout as qkv
  int* status;
};

constexpr int FB128_THREADS = 512;  // WG0: TMA + MMA, WG1/WG2: softmax halves, WG3: drain
constexpr int FB128_KV = 128;       // kv rows per CTA
constexpr int FB128_QT = 64;        // query rows per step
constexpr int FB128_D = 128;
constexpr int FB128_QS = 3;         // Q / dO stages

struct FaBwd128Smem {
  static constexpr int KV_TILE = FB128_KV * FB128_D * 2;     // 32 KB: two blocks of 128 rows x 128 B
  static constexpr int Q_TILE = FB128_QT * FB128_D * 2;      // 16 KB: two blocks of 64 rows x 128 B
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = KV_TILE;
  static constexpr int QDO_OFF = 2 * KV_TILE;                        // QS x (Q tile, dO tile)
  static constexpr int DS_OFF = QDO_OFF + FB128_QS * 2 * Q_TILE;     // dS^T: 128 kv rows x 64 q bf16
  static constexpr int DQ_OFF = DS_OFF + 16384;                      // dQ staging: 8 boxes of 32 x 32 fp32
  static constexpr int STAT_OFF = DQ_OFF + 32768;                    // QS x (-lse2[64], -delta[64])
  static constexpr int BAR_OFF = STAT_OFF + FB128_QS * 512;
  static constexpr int TOTAL = BAR_OFF + 512;                        // base must come 1024-byte aligned
};

__device__ __forceinline__ void kv128_red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b),
               "f"(c), "f"(d)
               : "memory");
}

__global__ void __launch_bounds__(FB128_THREADS, 1)
fa_bwd_kv128_kernel(const __grid_constant__ CUtensorMap tm_kv,    // qkv, boxes of 128 rows x 64 cols
                    const __grid_constant__ CUtensorMap tm_q,     // qkv, boxes of 64 rows x 64 cols
                    const __grid_constant__ CUtensorMap tm_do,    // dout, boxes of 64 rows x 64 cols
                    const __grid_constant__ CUtensorMap tm_acc,   // accumulator, 32 x 32 fp32 boxes
                    const FaBwd128Params p) {
  using L = FaBwd128Smem;
  constexpr int D = FB128_D, QS = FB128_QS;
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
  uint64_t* s_free = bars + 10;      // (count 256) ... and in registers
  uint64_t* dp_full = bars + 11;     // dP^T of a step is in TMEM
  uint64_t* dp_free = bars + 12;     // (count 256) ... and in registers
  uint64_t* p_ready = bars + 13;     // (count 256) P^T of a step is stored in TMEM
  uint64_t* p_free = bars + 14;      // dV has read it
  uint64_t* pds_ready = bars + 15;   // (count 256) dS^T of a step is stored (TMEM + smem)
  uint64_t* dst_free = bars + 16;    // dK has read dS^T from TMEM
  uint64_t* ds_free = bars + 17;     // dQ^T has read the shared-memory dS^T tile
  uint64_t* dq_full = bars + 18;     // 1
  uint64_t* dq_drained = bars + 19;  // 1 (count 128)
  uint64_t* dkv_full = bars + 20;    // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 22);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = warp_idx_uniform();
  const int lane = threadIdx.x & 31;

  // work decomposition: kv tile ascending = heavy first
  const int chunks = p.g / p.hpc;
  int bid = blockIdx.x;
  const int hc = bid % chunks; bid /= chunks;
  const int grp = bid % p.n_groups; bid /= p.n_groups;
  const int b = bid % p.batch; bid /= p.batch;
  const int j = bid;  // kv tile
  const int k_col = (grp * (p.g + 2) + p.g) * D;
  const int v_col = k_col + D;
  const int row_base = b * p.S;
  const int qt0 = 2 * j;                         // first 64-row query tile that sees this kv tile
  const int n_q = p.S / FB128_QT - qt0;          // query tiles qt0 .. S/64-1
  const int N = p.hpc * n_q;                     // steps of this CTA

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
    mbar_init(pds_ready, 256);
    mbar_init(dst_free, 1);
    mbar_init(ds_free, 1);
    mbar_init(dq_full, 1);
    mbar_init(dq_drained, 128);
    mbar_init(dkv_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tm_kv);
    prefetch_tmap(&tm_q);
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
  const uint32_t tm_S = tmem_base;
  const uint32_t tm_dP = tmem_base + 64;
  const uint32_t tm_dV = tmem_base + 128;
  const uint32_t tm_dK = tmem_base + 256;
  const uint32_t tm_dQ = tmem_base + 384;
  const uint32_t tm_Pt = tmem_base + 448;
  const uint32_t tm_dSt = tmem_base + 480;

  // step n -> (head, 64-row query tile)
  auto step_head = [&](int n) { return grp * p.g + hc * p.hpc + n / n_q; };
  auto step_qtile = [&](int n) { return qt0 + n % n_q; };

  if (warp < 4) {
  reg_dealloc<88>();
  if (warp == 0) {
    // ---------------- producer: one load per lane ----------------
    if (lane < 6) {
      if (lane == 0) mbar_expect_tx(kv_full, 2 * L::KV_TILE);
      if (lane < 4) {
        // K block 0 / 1, V block 0 / 1: 128 rows x 64 columns each
        uint8_t* dst = smem + (lane < 2 ? L::K_OFF : L::V_OFF) + (lane & 1) * 16384;
        tma_load_2d(dst, &tm_kv, kv_full, (lane < 2 ? k_col : v_col) + (lane & 1) * 64,
                    row_base + j * FB128_KV);
      }
      for (int n = 0; n < N; ++n) {
        const int s = n % QS;
        const int head = step_head(n), qt = step_qtile(n);
        const int q_col = (grp * (p.g + 2) + head % p.g) * D;
        mbar_wait_relaxed(&qdo_empty[s], ((n / QS) & 1) ^ 1, abort_flag, p.status, FT_ERR_WAIT_EMPTY);
        if (lane == 0) mbar_expect_tx(&qdo_full[s], 2 * L::Q_TILE + 512);
        uint8_t* dst = smem + L::QDO_OFF + s * 2 * L::Q_TILE;
        const int y = row_base + qt * FB128_QT;
        if (lane < 2) {
          tma_load_2d(dst + lane * 8192, &tm_q, &qdo_full[s], q_col + lane * 64, y);
        } else if (lane < 4) {
          tma_load_2d(dst + L::Q_TILE + (lane - 2) * 8192, &tm_do, &qdo_full[s],
                      head * D + (lane - 2) * 64, y);
        } else {
          // the statistics rows live and die with the Q / dO stage
          const long soff = (static_cast<long>(b) * p.Hq + head) * p.S + qt * FB128_QT;
          float* st = reinterpret_cast<float*>(smem + L::STAT_OFF + s * 512);
          if (lane == 4)
            bulk_load_1d(st, p.lse2 + soff, 256, &qdo_full[s]);
          else
            bulk_load_1d(st + 64, p.delta + soff, 256, &qdo_full[s]);
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
    const uint32_t idesc_s = make_idesc_bf16(128, FB128_QT, 0, 0);    // K-major x K-major, N = 64
    const uint32_t idesc_t = make_idesc_bf16(128, D, 0, 1);           // A from TMEM, B MN-major, N = 128
    const uint32_t idesc_dq = make_idesc_bf16(128, FB128_QT, 1, 1);   // K^T (MN-major) x dS^T (MN-major)
    const uint32_t sK = smem_u32(smem + L::K_OFF), sV = smem_u32(smem + L::V_OFF);
    const uint32_t sQDO = smem_u32(smem + L::QDO_OFF), sDS = smem_u32(smem + L::DS_OFF);
    // K-major operand of R rows x 128 columns = two blocks of R x 64: reduction step kk (16
    // elements) sits at (kk/4) * (R*128) + (kk%4)*32 bytes. MN-major operand: reduction step kk
    // (16 rows of 128 B) at kk*2048 bytes, 64-wide blocks of the other index LBO bytes apart.
    const uint32_t kK = smem_desc_lo(sK, 16), vK = smem_desc_lo(sV, 16);
    const uint32_t kMN = smem_desc_lo(sK, 16384);          // K^T as A: M = d over two blocks
    const uint32_t qK0 = smem_desc_lo(sQDO, 16);           // Q / dO as K-major B (N = 64 rows)
    const uint32_t qMN0 = smem_desc_lo(sQDO, 8192);        // Q / dO as MN-major B: N = d over two blocks
    const uint32_t dsMN = smem_desc_lo(sDS, 16384);        // dS^T as MN-major B: N = q, one block
    constexpr uint32_t STG = (2 * L::Q_TILE) >> 4, TL = L::Q_TILE >> 4;
#define FT_KOFF128(kk) ((((kk) / 4) * 16384 + ((kk) % 4) * 32) >> 4)
#define FT_KOFF64(kk) ((((kk) / 4) * 8192 + ((kk) % 4) * 32) >> 4)
#define FT_MNOFF(kk) (((kk) * 2048) >> 4)
    auto wait_qdo = [&](int n) {
      mbar_wait(&qdo_full[n % QS], (n / QS) & 1, abort_flag, p.status, FT_ERR_WAIT_FULL);
      tc_fence_after();
    };
    auto issue_s = [&](int n) {            // S^T = K Q^T
      const uint32_t qK = qK0 + (n % QS) * STG;
      umma_ss_lo<0>(tm_S, kK, qK, idesc_s);
#pragma unroll
      for (int kk = 1; kk < D / 16; ++kk)
        umma_ss_lo<1>(tm_S, kK + FT_KOFF128(kk), qK + FT_KOFF64(kk), idesc_s);
      umma_commit(s_full);
    };
    auto issue_dp = [&](int n) {           // dP^T = V dO^T
      const uint32_t doK = qK0 + (n % QS) * STG + TL;
      umma_ss_lo<0>(tm_dP, vK, doK, idesc_s);
#pragma unroll
      for (int kk = 1; kk < D / 16; ++kk)
        umma_ss_lo<1>(tm_dP, vK + FT_KOFF128(kk), doK + FT_KOFF64(kk), idesc_s);
      umma_commit(dp_full);
    };
    auto issue_dv = [&](int n) {           // dV += P^T dO, A from TMEM, K = 64 query rows
      const uint32_t doMN = qMN0 + (n % QS) * STG + TL;
      umma_ts_lo_dyn(tm_dV, tm_Pt, doMN, idesc_t, n > 0 ? 1u : 0u);
#pragma unroll
      for (int kk = 1; kk < FB128_QT / 16; ++kk)
        umma_ts_lo<1>(tm_dV, tm_Pt + kk * 8, doMN + FT_MNOFF(kk), idesc_t);
      umma_commit(p_free);
    };
    auto issue_dk = [&](int n) {           // dK += dS^T Q, A from TMEM
      const uint32_t qMN = qMN0 + (n % QS) * STG;
      umma_ts_lo_dyn(tm_dK, tm_dSt, qMN, idesc_t, n > 0 ? 1u : 0u);
#pragma unroll
      for (int kk = 1; kk < FB128_QT / 16; ++kk)
        umma_ts_lo<1>(tm_dK, tm_dSt + kk * 8, qMN + FT_MNOFF(kk), idesc_t);
      umma_commit(dst_free);
      // Q_n / dO_n are last read by dK / dV: hand the stage back to the producer now
      umma_commit(&qdo_empty[n % QS]);
    };
    auto issue_dq = [&](int n) {           // dQ^T = K^T dS^T, K = 128 kv rows
      umma_ss_lo<0>(tm_dQ, kMN, dsMN, idesc_dq);
#pragma unroll
      for (int kk = 1; kk < FB128_KV / 16; ++kk)
        umma_ss_lo<1>(tm_dQ, kMN + FT_MNOFF(kk), dsMN + FT_MNOFF(kk), idesc_dq);
      umma_commit(dq_full);
      umma_commit(ds_free);
    };
    mbar_wait(kv_full, 0, abort_flag, p.status, FT_ERR_WAIT_FULL);
    wait_qdo(0);
    if (elect_one_sync()) {
      issue_s(0);
      issue_dp(0);
    }
    __syncwarp();
    for (int n = 0; n < N; ++n) {
      mbar_wait(p_ready, n & 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
      tc_fence_after();
      if (elect_one_sync()) issue_dv(n);
      __syncwarp();
      if (n + 1 < N) {
        // the next step's S^T / dP^T as soon as this step's are in registers
        mbar_wait(s_free, n & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_EMPTY);
        wait_qdo(n + 1);
        if (elect_one_sync()) issue_s(n + 1);
        __syncwarp();
        mbar_wait(dp_free, n & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_EMPTY);
        tc_fence_after();
        if (elect_one_sync()) issue_dp(n + 1);
        __syncwarp();
      }
      mbar_wait(pds_ready, n & 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
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
#undef FT_KOFF128
#undef FT_KOFF64
#undef FT_MNOFF
    if (elect_one_sync()) umma_commit(dkv_full);
    __syncwarp();
  }
  } else if (warp < 12) {
    reg_alloc<152>();
    // ---------------- two softmax warpgroups: thread owns kv row r and 32 of the 64 query
    // columns of a step (warpgroup 1: columns 0-31, warpgroup 2: columns 32-63) ----------------
    const int half = (warp - 4) >> 2;
    const int r = (threadIdx.x - 128) & 127;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint64_t sl2x2 = pack_f32x2(p.scale_log2, p.scale_log2);
    uint8_t* rowd = smem + L::DS_OFF + r * 128;   // this thread's dS^T row (64 q = 128 B)
    for (int n = 0; n < N; ++n) {
      const int qt = step_qtile(n);
      const float4* nl4 = reinterpret_cast<const float4*>(smem + L::STAT_OFF + (n % QS) * 512) + half * 8;
      const float4* nd4 = nl4 + 16;
      mbar_wait(&qdo_full[n % QS], (n / QS) & 1, abort_flag, p.status, FT_ERR_WAIT_FULL);
      mbar_wait(s_full, n & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_FULL);
      tc_fence_after();
      alignas(8) uint32_t s[32];
      tmem_ld32(tm_S + lane_off + half * 32, s);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(s_free);
      if (qt < qt0 + 2) {  // the two query tiles on the diagonal: query position < kv position is masked
        const int qbase = (qt - qt0) * FB128_QT + half * 32;
#pragma unroll
        for (int k = 0; k < 32; ++k)
          if (qbase + k < r) s[k] = 0xff800000u;  // -inf -> p = 0
      }
      uint64_t* s2 = reinterpret_cast<uint64_t*>(s);    // pairs of scores, then probabilities
      uint32_t w[16];                                   // packed bf16 row piece (P^T, then dS^T)
#pragma unroll
      for (int c = 0; c < 8; ++c) {                     // P^T = exp2(S^T * scale - lse2)
        const float4 l = nl4[c];                        // -lse2 of four query columns
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
      tmem_st16(tm_Pt + lane_off + half * 16, w);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(p_ready);
      mbar_wait(dp_full, n & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_FULL);
      tc_fence_after();
      alignas(8) uint32_t dp[32];
      tmem_ld32(tm_dP + lane_off + half * 32, dp);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(dp_free);
      uint64_t* d2 = reinterpret_cast<uint64_t*>(dp);
#pragma unroll
      for (int c = 0; c < 8; ++c) {                     // dS^T = P^T * (dP^T - delta)
        const float4 dl = nd4[c];                       // -delta of four query columns
        const uint64_t x0 = mul_f32x2(s2[2 * c], add_f32x2(d2[2 * c], pack_f32x2(dl.x, dl.y)));
        const uint64_t x1 = mul_f32x2(s2[2 * c + 1], add_f32x2(d2[2 * c + 1], pack_f32x2(dl.z, dl.w)));
        float a0, a1, a2, a3;
        unpack_f32x2(x0, a0, a1);
        unpack_f32x2(x1, a2, a3);
        w[2 * c] = pack_bf16x2(a0, a1);
        w[2 * c + 1] = pack_bf16x2(a2, a3);
      }
      // dK of the previous step has read dS^T from TMEM; dQ^T of the previous step the smem tile
      if (n > 0) {
        mbar_wait(dst_free, (n - 1) & 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
        mbar_wait(ds_free, (n - 1) & 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
        tc_fence_after();
      }
      tmem_st16(tm_dSt + lane_off + half * 16, w);
#pragma unroll
      for (int c = 0; c < 4; ++c)
        *reinterpret_cast<uint4*>(rowd + (((half * 4 + c) ^ (r & 7)) << 4)) =
            make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
      tmem_st_wait();
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(pds_ready);
    }
  } else {
    reg_dealloc<88>();
    // ---------------- drain warpgroup. dQ^T every step: thread d owns head-dim index d and
    // holds the 64 query rows of the step; warp w stages its 32 columns as two swizzled boxes of
    // 32 query rows x 32 floats (the transposition happens in these stores: for one query row
    // the 32 lanes write 32 consecutive floats) and one lane sends them off as TMA reduce-adds.
    // dK / dV at the end: thread r owns kv row r. ----------------
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
      mbar_arrive(dq_drained);                 // in registers: dQ^T of the next step may start
      if (n > 0) {                             // the previous step's boxes have been read
        if (lane == 0) tma_wait_group_read<0>();
        __syncwarp();
      }
#pragma unroll
      for (int q = 0; q < 64; ++q)
        *reinterpret_cast<uint32_t*>(stage + (q >> 5) * 4096 + (q & 31) * 128 +
                                     ((((lane >> 2) ^ (q & 7)) << 4) | ((lane & 3) << 2))) = o[q];
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        const int y = row_base + qt * FB128_QT;
        tma_reduce_add_2d(&tm_acc, stage, q_col + q4 * 32, y);
        tma_reduce_add_2d(&tm_acc, stage + 4096, q_col + q4 * 32, y + 32);
        tma_commit_group();
      }
    }
    if (lane == 0) tma_wait_group<0>();
    __syncwarp();
    mbar_wait_relaxed(dkv_full, 0, abort_flag, p.status, FT_ERR_WAIT_TMEM_FULL, 256);
    tc_fence_after();
    float* acc_row = p.acc + static_cast<long>(row_base + j * FB128_KV + r) * p.ld_acc;
#pragma unroll 1
    for (int c = 0; c < D / 32; ++c) {
      uint32_t o[32];
      tmem_ld32(tm_dV + lane_off + c * 32, o);
      tmem_ld_wait();
#pragma unroll
      for (int k = 0; k < 8; ++k)
        kv128_red_add_v4(acc_row + v_col + c * 32 + 4 * k, __uint_as_float(o[4 * k]),
                         __uint_as_float(o[4 * k + 1]), __uint_as_float(o[4 * k + 2]),
                         __uint_as_float(o[4 * k + 3]));
      tmem_ld32(tm_dK + lane_off + c * 32, o);
      tmem_ld_wait();
#pragma unroll
      for (int k = 0; k < 8; ++k)
        kv128_red_add_v4(acc_row + k_col + c * 32 + 4 * k, __uint_as_float(o[4 * k]),
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

// Launch of the TMEM-operand main kernel (head_dim 128). `tkv`: qkv map with 128 x 64 boxes,
// `tq` / `tdo`: qkv / dout maps with 64 x 64 boxes, `tacc`: 32 x 32 fp32 boxes over the
// accumulator; `neg_lse2` / `neg_delta` hold the NEGATED statistics.
int launch_fa_bwd_kv128(const CUtensorMap& tkv, const CUtensorMap& tq, const CUtensorMap& tdo,
                        const CUtensorMap& tacc, int S, int Hq, int g, int n_groups, int batch,
                        int hpc, int ld_acc, float scale_log2, const float* neg_lse2,
                        const float* neg_delta, float* acc, int* status, cudaStream_t st) {
  using L = FaBwd128Smem;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(fa_bwd_kv128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             L::TOTAL) != cudaSuccess)
      return -10;
    attr = true;
  }
  FaBwd128Params p;
  p.S = S; p.Hq = Hq; p.g = g; p.n_groups = n_groups; p.batch = batch; p.hpc = hpc;
  p.ld_acc = ld_acc;
  p.scale_log2 = scale_log2;
  p.lse2 = neg_lse2; p.delta = neg_delta; p.acc = acc;
  p.status = status;
  const int grid = (S / FB128_KV) * batch * n_groups * (g / hpc);
  fa_bwd_kv128_kernel<<<grid, FB128_THREADS, L::TOTAL, st>>>(tkv, tq, tdo, tacc, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace ft
