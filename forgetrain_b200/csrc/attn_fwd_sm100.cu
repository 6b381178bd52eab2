// Causal GQA FlashAttention forward for sm_100a (head_dim 64 or 128), reading q/k/v straight out
// of the interleaved projection buffer qkv[T][n_groups*(g+2)*D] through strided TMA boxes and
// writing out[T][Hq*D] plus the log-sum-exp.
//
// One CTA owns two consecutive 128-row query tiles of one (batch, head) and ping-pongs them:
//   warp 0      TMA producer  (Q once, then K_j / V_j rings)
//   warps 1, 2  MMA issuers, one per query tile (tcgen05.mma: S_w = Q_w K_j^T, O_w += P_w V_j;
//               TMEM accumulators)
//   warps 4-7   softmax of tile 0 (one thread per query row, no shuffles)
//   warps 8-11  softmax of tile 1
// While one warpgroup exponentiates, the tensor core works for the other tile. The running
// maximum is only refreshed when it grew by more than 2^8 ("lazy rescale"), which keeps the
// TMEM round-trip of O off the common path. At head_dim 64 the probabilities never touch shared
// memory: the softmax threads store them (packed bf16) into 64 TMEM columns per tile and the
// P V product reads its A operand from there, which takes 64 KB of shared-memory traffic per
// 128 x 128 score block off the busiest pipe of this kernel. At head_dim 128 S and O fill all
// 512 columns, so P goes through shared memory in the 128-byte swizzled K-major layout.
//
// One warp can issue an `ex2` only every ~16 cycles, whatever else is ready, so the exponentials
// are not a stage of their own: scale, exponential (one pair in four by polynomial on the FMA
// pipe), row-sum and bf16 packing are one interleaved stream over 8-column chunks, and the other
// instructions issue in the gaps between two `ex2`.
//
// Replaces the reference's Hopper FlashAttention forward kernels
// (ops/attention/flash_attn_dsl/flash_fwd.py:31-660, src/flash_attn_dsl/flash_fwd.py:1-803).
#include "ptx.cuh"
#include "tma_host.h"

namespace ft {

int get_tmap_2d(CUtensorMap* out, const void* base, int elt, uint64_t rows, uint64_t cols,
                uint64_t ld, uint32_t box_r, uint32_t box_c);
int launch_fa_fwd1(const CUtensorMap& tq, const CUtensorMap& to, int D, int S, int Hq, int g,
                   int n_groups, int batch, float scale_log2, float* lse, int* status,
                   cudaStream_t st);

constexpr int FA_THREADS = 384;
constexpr int FA_BLK = 128;
// Pairs out of every 4 whose 2^x is evaluated by polynomial on the FMA pipe instead of the
// transcendental unit (measured optimum: one at head_dim 64, none at 128, where the shared-
// memory stores of P already fill the issue slots between two `ex2`).
#ifndef FA_POLY
#define FA_POLY(D) ((D) == 64 ? 1 : 0)
#endif
#ifndef FA_REG_SOFTMAX
#define FA_REG_SOFTMAX 200
#define FA_REG_CONTROL 96
#endif
#ifndef FT_FA_FWD1_D128
#define FT_FA_FWD1_D128 1   // head_dim 128 on the one-tile kernel as well
#endif
#ifndef FA_PACK
#define FA_PACK pack_bf16x2   // fp32 pair -> packed bf16 (cvt), or pack_bf16x2_int (integer pipe)
#endif

struct FaFwdParams {
  int S, Hq, g, n_groups, batch;
  float scale_log2;  // softmax scale * log2(e)
  float* lse;        // [B][Hq][S]
  int* status;
};

template <int D, int KS, int VS>
struct FaFwdSmem {
  static constexpr bool P_TMEM = D == 64;            // P lives in TMEM (room only at head_dim 64)
  static constexpr int TILE = FA_BLK * D * 2;        // one 128 x D bf16 tile
  static constexpr int Q_OFF = 0;                    // 2 tiles
  static constexpr int K_OFF = 2 * TILE;
  static constexpr int V_OFF = K_OFF + KS * TILE;
  static constexpr int P_OFF = V_OFF + VS * TILE;    // 2 x (128 x 128 bf16) unless P_TMEM
  static constexpr int BAR_OFF = P_OFF + (P_TMEM ? 0 : 2 * 32768);
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

template <int D, int KS, int VS>
__global__ void __launch_bounds__(FA_THREADS, 1)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_out,
              const FaFwdParams p) {
  using L = FaFwdSmem<D, KS, VS>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  static_assert(KS <= 4 && VS <= 4, "four barrier slots per ring");
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // KS (<= 4)
  uint64_t* k_empty = bars + 5;
  uint64_t* v_full = bars + 9;        // VS (<= 4)
  uint64_t* v_empty = bars + 13;
  uint64_t* s_full = bars + 17;       // 2
  uint64_t* p_ready = bars + 19;      // 2
  uint64_t* o_done = bars + 21;       // 2
  uint64_t* s_free = bars + 23;       // 2 (count 128): the score row of a step is in registers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 26);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = warp_idx_uniform();
  const int lane = threadIdx.x & 31;

  // heavy (late) query tiles first; heads of one KV group adjacent for L2 reuse of K/V
  const int n_pairs = p.S / (2 * FA_BLK);
  const int head = blockIdx.x % p.Hq;
  const int rest = blockIdx.x / p.Hq;
  const int b = rest % p.batch;
  const int pair = n_pairs - 1 - rest / p.batch;
  const int grp = head / p.g;
  const int q_col = (grp * (p.g + 2) + head % p.g) * D;
  const int k_col = (grp * (p.g + 2) + p.g) * D;
  const int v_col = k_col + D;
  const int row_base = b * p.S;
  const int n_kv[2] = {2 * pair + 1, 2 * pair + 2};
  const int n_total = n_kv[1];

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 4; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 2);   // one commit from each of the two issuing threads
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 2);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&p_ready[s], 128);
      mbar_init(&o_done[s], 1);
      mbar_init(&s_free[s], 128);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tm_qkv);
    prefetch_tmap(&tm_out);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S[2] = {tmem_base, tmem_base + 128};
  const uint32_t tmem_O[2] = {tmem_base + 256, tmem_base + 256 + D};
  const uint32_t tmem_P[2] = {tmem_base + 384, tmem_base + 448};   // P_TMEM only (D == 64)

  if (warp < 4) {
  reg_dealloc<FA_REG_CONTROL>();   // TMA / MMA warps need few registers, the softmax warps a whole score row
  if (warp == 0) {
    // ---------------- producer: lanes [0, NBOX) load K, lanes [NBOX, 2 NBOX) load V, one
    // 64-column box each (a thread that issues a TMA load is held for several hundred cycles
    // per instruction, so the boxes of a step go out from different lanes) ----------------
    constexpr int NBOX = D / 64;
    if (lane < 2 * NBOX) {
      const int c = lane % NBOX;
      const bool is_v = lane >= NBOX;
      if (lane == 0) mbar_expect_tx(q_full, 2 * L::TILE);
      // Q tiles: 2 * NBOX boxes, one per lane
      {
        const int w = lane / NBOX;
        tma_load_2d(smem + L::Q_OFF + w * L::TILE + c * 16384, &tm_qkv, q_full, q_col + c * 64,
                    row_base + (2 * pair + w) * FA_BLK);
      }
      for (int j = 0; j < n_total; ++j) {
        if (!is_v) {
          const int ks = j % KS;
          mbar_wait(&k_empty[ks], ((j / KS) & 1) ^ 1, abort_flag, p.status, FT_ERR_WAIT_EMPTY);
          if (c == 0) mbar_expect_tx(&k_full[ks], L::TILE);
          tma_load_2d(smem + L::K_OFF + ks * L::TILE + c * 16384, &tm_qkv, &k_full[ks],
                      k_col + c * 64, row_base + j * FA_BLK);
        } else {
          const int vs = j % VS;
          mbar_wait(&v_empty[vs], ((j / VS) & 1) ^ 1, abort_flag, p.status, FT_ERR_WAIT_EMPTY);
          if (c == 0) mbar_expect_tx(&v_full[vs], L::TILE);
          tma_load_2d(smem + L::V_OFF + vs * L::TILE + c * 16384, &tm_qkv, &v_full[vs],
                      v_col + c * 64, row_base + j * FA_BLK);
        }
      }
      if (lane == 0 && *abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1 || warp == 2) {
    {
      // ---------------- MMA issuers: warp 1 serves query tile 0, warp 2 tile 1 ----------------
      // Each tile has its own in-order chain S(0), [S(j+1), P V(j)]...; one thread per tile
      // sleeps on exactly the barrier its chain needs next, so neither tile ever waits for the
      // other warpgroup's softmax. The tensor pipe takes the two threads' products in arrival
      // order. A K / V stage goes back to the producer when both threads have committed it.
      // The whole warp runs the loop and the waits; one elected lane issues.
      const int w = warp - 1;
      const int nk = n_kv[w];
      const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_o = make_idesc_bf16(128, D, 0, 1);
      const uint32_t sQ = smem_u32(smem + L::Q_OFF), sK = smem_u32(smem + L::K_OFF);
      const uint32_t sV = smem_u32(smem + L::V_OFF), sP = smem_u32(smem + L::P_OFF);
      // descriptor low words: K-major step kk: +(kk/4)*16384 + (kk%4)*32 bytes; MN-major: + kk*2048
      constexpr uint32_t TL = L::TILE >> 4, PB = 32768 >> 4;
      const uint32_t qa = smem_desc_lo(sQ, 16) + w * TL, kK0 = smem_desc_lo(sK, 16);
      const uint32_t pa = smem_desc_lo(sP, 16) + w * PB, vMN0 = smem_desc_lo(sV, 16384);
      (void)pa;
      const uint32_t tS = tmem_S[w], tO = tmem_O[w], tP = tmem_P[w];
      (void)tP;
#define FT_KOFF(kk) ((((kk) / 4) * 16384 + ((kk) % 4) * 32) >> 4)
#define FT_MNOFF(kk) (((kk) * 2048) >> 4)
      auto issue_S = [&](int j) {
        const uint32_t ka = kK0 + (j % KS) * TL;
        umma_ss_lo<0>(tS, qa, ka, idesc_s);
#pragma unroll
        for (int kk = 1; kk < D / 16; ++kk)
          umma_ss_lo<1>(tS, qa + FT_KOFF(kk), ka + FT_KOFF(kk), idesc_s);
        umma_commit(&s_full[w]);
        umma_commit(&k_empty[j % KS]);
      };
      auto issue_PV = [&](int j) {
        const uint32_t va = vMN0 + (j % VS) * TL;
        if constexpr (L::P_TMEM) {
          umma_ts_lo_dyn(tO, tP, va, idesc_o, j > 0 ? 1u : 0u);
#pragma unroll
          for (int kk = 1; kk < 8; ++kk)   // 16 bf16 of a row = 8 TMEM columns per k-step
            umma_ts_lo<1>(tO, tP + kk * 8, va + FT_MNOFF(kk), idesc_o);
        } else {
          umma_ss_lo_dyn(tO, pa, va, idesc_o, j > 0 ? 1u : 0u);
#pragma unroll
          for (int kk = 1; kk < 8; ++kk)
            umma_ss_lo<1>(tO, pa + FT_KOFF(kk), va + FT_MNOFF(kk), idesc_o);
        }
        umma_commit(&o_done[w]);
        umma_commit(&v_empty[j % VS]);
      };
      mbar_wait(q_full, 0, abort_flag, p.status, FT_ERR_WAIT_FULL);
      mbar_wait(&k_full[0], 0, abort_flag, p.status, FT_ERR_WAIT_FULL);
      tc_fence_after();
      if (elect_one_sync()) issue_S(0);
      __syncwarp();
      for (int j = 0; j < nk; ++j) {
        // S of step j+1 goes to the tensor pipe as soon as the softmax warpgroup holds the
        // score row of step j in registers, i.e. while it is still exponentiating it.
        if (j + 1 < nk) {
          mbar_wait(&s_free[w], j & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_EMPTY);
          mbar_wait(&k_full[(j + 1) % KS], ((j + 1) / KS) & 1, abort_flag, p.status,
                    FT_ERR_WAIT_FULL);
          tc_fence_after();
          if (elect_one_sync()) {
            issue_S(j + 1);
          }
          __syncwarp();
        }
        mbar_wait(&v_full[j % VS], (j / VS) & 1, abort_flag, p.status, FT_ERR_WAIT_FULL);
        mbar_wait(&p_ready[w], j & 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
        tc_fence_after();
        if (elect_one_sync()) {
          issue_PV(j);
        }
        __syncwarp();
      }
    }
  }
#undef FT_KOFF
#undef FT_MNOFF
  } else {
    reg_alloc<FA_REG_SOFTMAX>();
    // ---------------- softmax warpgroups ----------------
    const int w = (warp - 4) >> 2;           // query tile of this warpgroup
    const int r = threadIdx.x - 128 - w * 128;  // row inside the tile == TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int qt = 2 * pair + w;
    const int q_row = qt * FA_BLK + r;  // position inside the sequence
    uint8_t* sP = smem + L::P_OFF + w * 32768;   // unused when P lives in TMEM
    // staging of the output tile: the P buffer, or (P in TMEM) this tile's Q buffer, which the
    // tensor core has finished reading once the last score block of the tile is in registers
    uint8_t* sO = L::P_TMEM ? smem + L::Q_OFF + w * L::TILE : sP;
    float m_ref = -INFINITY, l = 0.f;
    const int nk = n_kv[w];
    const uint64_t sl2x2 = pack_f32x2(p.scale_log2, p.scale_log2);
    uint64_t lsum2 = pack_f32x2(0.f, 0.f);
    for (int j = 0; j < nk; ++j) {
      mbar_wait(&s_full[w], j & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_FULL);
      tc_fence_after();
      // one pass over TMEM: the whole score row (128 fp32) lives in registers
      alignas(8) uint32_t s[128];
      tmem_ld32(tmem_S[w] + lane_off, s);
      tmem_ld32(tmem_S[w] + lane_off + 32, s + 32);
      tmem_ld32(tmem_S[w] + lane_off + 64, s + 64);
      tmem_ld32(tmem_S[w] + lane_off + 96, s + 96);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&s_free[w]);
      if (j == qt) {  // diagonal tile: columns beyond the row are masked
#pragma unroll
        for (int k = 0; k < 128; ++k)
          if (k > r) s[k] = 0xff800000u;  // -inf
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int k = 0; k < 128; k += 8) {   // four independent chains of 16
        mx0 = max3(mx0, __uint_as_float(s[k]), __uint_as_float(s[k + 1]));
        mx1 = max3(mx1, __uint_as_float(s[k + 2]), __uint_as_float(s[k + 3]));
        mx2 = max3(mx2, __uint_as_float(s[k + 4]), __uint_as_float(s[k + 5]));
        mx3 = max3(mx3, __uint_as_float(s[k + 6]), __uint_as_float(s[k + 7]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      const float m_new = fmaxf(m_ref, mx * p.scale_log2);
      const bool need = (m_new - m_ref) > 8.0f;  // also true while m_ref is still -inf
      bool o_waited = false;
      if (__any_sync(0xffffffffu, need)) {
        if (j > 0) {   // the rescale touches O: the previous P V product must have landed
          mbar_wait(&o_done[w], (j - 1) & 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
          tc_fence_after();
          o_waited = true;
        }
        const float alpha = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - m_new);
        m_ref = m_new;
        lsum2 = mul_f32x2(lsum2, pack_f32x2(alpha, alpha));
        if (j > 0) {
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(tmem_O[w] + lane_off + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int k = 0; k < 32; ++k) o[k] = __float_as_uint(__uint_as_float(o[k]) * alpha);
            tmem_st32(tmem_O[w] + lane_off + c * 32, o);
          }
          tmem_st_wait();
        }
      }
      const uint64_t negm2 = pack_f32x2(-m_ref, -m_ref);
      // One interleaved stream over 16 chunks of 8 columns: scale, exponential (FA_POLY pairs of
      // every 4 by polynomial on the FMA pipe), row sum, bf16 packing. Two softmax warps share a
      // scheduler's transcendental unit (one `ex2` per ~8 cycles); everything else goes out in
      // between.
      uint64_t* s2 = reinterpret_cast<uint64_t*>(s);
      uint64_t acc0 = pack_f32x2(0.f, 0.f), acc1 = acc0, acc2 = acc0, acc3 = acc0;
      // P in TMEM: the packed probabilities stay in registers until the stream is over (they
      // take the place of the scores they were made from) and are stored in one go afterwards.
      // The P columns are still being read by the previous P V product when the stream starts;
      // waiting for that product BEFORE the stream left the warpgroup idle while the product sat
      // in the tensor pipe's queue behind the other query tile's work (0.222 -> 0.211 ms). P in
      // shared memory (head_dim 128): the same deferral measured slower (0.141 -> 0.145 ms, the
      // 16 stores leave in one burst), so there the wait comes first and the stores go out with
      // the stream.
      uint32_t pk[L::P_TMEM ? 64 : 4];
      if constexpr (!L::P_TMEM) {
        if (j > 0 && !o_waited) {
          mbar_wait(&o_done[w], (j - 1) & 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
          tc_fence_after();
        }
      }
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        uint32_t w4[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int i = c * 4 + q;
          uint64_t t = fma_f32x2(s2[i], sl2x2, negm2);
          float e0, e1;
          if (q < FA_POLY(D)) {
            t = exp2_poly_f32x2(t);
            unpack_f32x2(t, e0, e1);
          } else {
            unpack_f32x2(t, e0, e1);
            e0 = fast_exp2(e0);
            e1 = fast_exp2(e1);
            t = pack_f32x2(e0, e1);
          }
          if (q == 0) acc0 = add_f32x2(acc0, t);
          else if (q == 1) acc1 = add_f32x2(acc1, t);
          else if (q == 2) acc2 = add_f32x2(acc2, t);
          else acc3 = add_f32x2(acc3, t);
          w4[q] = FA_PACK(e0, e1);
        }
        if constexpr (L::P_TMEM) {
#pragma unroll
          for (int q = 0; q < 4; ++q) pk[c * 4 + q] = w4[q];
        } else {
          uint8_t* rowp = sP + (c >> 3) * 16384 + r * 128;
          *reinterpret_cast<uint4*>(rowp + (((c & 7) ^ (r & 7)) << 4)) =
              make_uint4(w4[0], w4[1], w4[2], w4[3]);
        }
      }
      lsum2 = add_f32x2(lsum2, add_f32x2(add_f32x2(acc0, acc1), add_f32x2(acc2, acc3)));
      if constexpr (L::P_TMEM) {
        if (j > 0 && !o_waited) {   // the previous P V product has finished reading the P columns
          mbar_wait(&o_done[w], (j - 1) & 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
          tc_fence_after();
        }
        tmem_st32(tmem_P[w] + lane_off, pk);
        tmem_st32(tmem_P[w] + lane_off + 32, pk + 32);
        tmem_st_wait();
        tc_fence_before();
      } else {
        tc_fence_before();
        fence_proxy_async_smem();
      }
      mbar_arrive(&p_ready[w]);
    }
    {
      float l0, l1;
      unpack_f32x2(lsum2, l0, l1);
      l = l0 + l1;
    }
    // ---------------- epilogue: O / l -> bf16 -> TMA store; LSE ----------------
    mbar_wait(&o_done[w], (nk - 1) & 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
    tc_fence_after();
    const float inv_l = 1.f / l;
#pragma unroll 1
    for (int c = 0; c < D / 32; ++c) {
      uint32_t o[32];
      tmem_ld32(tmem_O[w] + lane_off + c * 32, o);
      tmem_ld_wait();
      uint8_t* rowp = sO + (c >> 1) * 16384 + r * 128;
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        uint4 u;
        u.x = pack_bf16x2(__uint_as_float(o[8 * jj + 0]) * inv_l, __uint_as_float(o[8 * jj + 1]) * inv_l);
        u.y = pack_bf16x2(__uint_as_float(o[8 * jj + 2]) * inv_l, __uint_as_float(o[8 * jj + 3]) * inv_l);
        u.z = pack_bf16x2(__uint_as_float(o[8 * jj + 4]) * inv_l, __uint_as_float(o[8 * jj + 5]) * inv_l);
        u.w = pack_bf16x2(__uint_as_float(o[8 * jj + 6]) * inv_l, __uint_as_float(o[8 * jj + 7]) * inv_l);
        const int chunk = (c & 1) * 4 + jj;
        *reinterpret_cast<uint4*>(rowp + ((chunk ^ (r & 7)) << 4)) = u;
      }
    }
    p.lse[(static_cast<long>(b) * p.Hq + head) * p.S + q_row] =
        (m_ref + log2f(l)) * 0.6931471805599453f;
    fence_proxy_async_smem();
    named_bar_sync(1 + w, 128);
    if (r == 0) {
#pragma unroll
      for (int c = 0; c < D / 64; ++c)
        tma_store_2d(&tm_out, sO + c * 16384, head * D + c * 64, row_base + qt * FA_BLK);
      tma_commit_group();
      tma_wait_group<0>();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int D, int KS, int VS>
static int launch_fa_fwd(const CUtensorMap& tq, const CUtensorMap& to, const FaFwdParams& p,
                         cudaStream_t st) {
  using L = FaFwdSmem<D, KS, VS>;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(fa_fwd_kernel<D, KS, VS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             L::TOTAL) != cudaSuccess)
      return -10;
    attr = true;
  }
  const int grid = (p.S / (2 * FA_BLK)) * p.batch * p.Hq;
  fa_fwd_kernel<D, KS, VS><<<grid, FA_THREADS, L::TOTAL, st>>>(tq, to, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace ft

// qkv: [batch*S][ld_qkv] bf16 interleaved per KV group as [q_0..q_{g-1} | k | v]; out:
// [batch*S][ld_out] bf16 with head h at columns [h*D, (h+1)*D); lse: [batch][Hq][S] fp32
// (natural log). S must be a multiple of 256, D 64 or 128.
extern "C" int ft_attn_fwd(const void* qkv, void* out, void* lse, int batch, int S, int n_groups,
                           int g, int D, int ld_qkv, int ld_out, float scale, int* status,
                           cudaStream_t st) {
  using namespace ft;
  if (S % (2 * FA_BLK) || (D != 64 && D != 128)) return -1;
  const long T = static_cast<long>(batch) * S;
  CUtensorMap tq, to;
  if (get_tmap_2d(&tq, qkv, 2, T, static_cast<uint64_t>(n_groups) * (g + 2) * D, ld_qkv, FA_BLK, 64))
    return -2;
  if (get_tmap_2d(&to, out, 2, T, static_cast<uint64_t>(n_groups) * g * D, ld_out, FA_BLK, 64))
    return -3;
  FaFwdParams p;
  p.S = S; p.Hq = n_groups * g; p.g = g; p.n_groups = n_groups; p.batch = batch;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.lse = static_cast<float*>(lse);
  p.status = status;
#ifndef FT_FA_FWD_TWO_TILES
  // one query tile per CTA, two CTAs per SM (attn_fwd1_sm100.cu)
  // (head_dim 128 at long sequences stays on the two-tile kernel: 0.450 vs 0.464 ms at S = 8192,
  // where the one-tile kernel's second copy of the K / V traffic shows; 0.137 vs 0.141 ms at 4096)
  if (D == 64 || (FT_FA_FWD1_D128 && S <= 4096))
    return launch_fa_fwd1(tq, to, D, S, p.Hq, g, n_groups, batch, p.scale_log2, p.lse, status, st);
#endif
  if (D == 64) return launch_fa_fwd<64, 3, 3>(tq, to, p, st);
  return launch_fa_fwd<128, 1, 1>(tq, to, p, st);   // the spare 32 KB as a second K stage measured slower (0.157 vs 0.141 ms), as a second V stage the same (0.143)
}
