// Causal GQA FlashAttention forward, ONE 128-row query tile per CTA and TWO CTAs per SM (head_dim
// 64, and head_dim 128 in the variant described at the end of this comment). Same arithmetic, layouts and softmax stream as attn_fwd_sm100.cu (P in TMEM, lazy rescale,
// one pair of exponentials in four by polynomial); what changes is who shares an SM. A CTA of that
// kernel ping-pongs two query tiles and owns all of TMEM, so an SM runs one CTA at a time and the
// launch of a CTA, its barrier / TMEM set-up, the first Q / K / V loads, the output pass and the
// tail all leave the tensor pipe and the transcendental unit idle: about 5 us for a work item of
// 20-60 us. Here a CTA takes 256 TMEM columns (S 128, O 64, P 64), 80 KB of shared memory and 256
// threads, so two of them are resident: the hardware overlaps one CTA's set-up and output with the
// other's steady state, and in steady state the two tiles share the tensor pipe as before.
//   warp 0      TMA producer (Q once, then the K_j / V_j rings)
//   warp 1      MMA issuer (S = Q K_j^T, O += P V_j)
//   warps 2, 3  idle (register reallocation works on whole warpgroups)
//   warps 4-7   softmax, one thread per query row
// head_dim 128: S (128 columns) and O (128) already fill the 256 columns, so the packed
// probabilities are written over the first 64 columns of S itself (every thread touches only its
// own TMEM lane, and its score row is in registers by then). The next score block can then only be
// issued behind the P V product that reads them (the tensor pipe runs one thread's products in
// order), so a CTA alternates softmax and tensor work, and the OTHER resident CTA fills the gaps.
// Shared memory: Q, one K and one V stage of 32 KB each.
#include "ptx.cuh"
#include "tma_host.h"

namespace ft {

constexpr int FA1_THREADS = 256;   // warpgroup 0: producer, issuer, two idle warps; warpgroup 1: softmax
constexpr int FA1_BLK = 128;
#ifndef FA1_POLY64
#define FA1_POLY64 1
#define FA1_POLY128 0
#endif
template <int D>
struct FaFwd1Cfg {
  static constexpr int STAGES = D == 64 ? 3 : 1;   // K and V stages
  static constexpr bool P_OVER_S = D == 128;       // P stored over the first 64 columns of S
  static constexpr int POLY = D == 64 ? FA1_POLY64 : FA1_POLY128;   // pairs in four whose 2^x goes to the FMA pipe
};

struct FaFwd1Params {
  int S, Hq, g, n_groups, batch;
  float scale_log2;  // softmax scale * log2(e)
  float* lse;        // [B][Hq][S]
  int* status;
};

template <int D>
struct FaFwd1Smem {
  static constexpr int TILE = FA1_BLK * D * 2;   // 16 / 32 KB, blocks of 128 rows x 64 columns
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = TILE;
  static constexpr int V_OFF = K_OFF + FaFwd1Cfg<D>::STAGES * TILE;
  static constexpr int BAR_OFF = V_OFF + FaFwd1Cfg<D>::STAGES * TILE;
  static constexpr int TOTAL = BAR_OFF + 256;   // base must come 1024-byte aligned (checked)
};

template <int D>
__global__ void __launch_bounds__(FA1_THREADS, 2)
fa_fwd1_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_out,
               const FaFwd1Params p) {
  using L = FaFwd1Smem<D>;
  using C = FaFwd1Cfg<D>;
  constexpr int KS = C::STAGES, VS = C::STAGES, NBOX = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023u) {  // swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, FT_ERR_WAIT_MISC);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // KS (<= 4)
  uint64_t* k_empty = bars + 5;
  uint64_t* v_full = bars + 9;        // VS (<= 4)
  uint64_t* v_empty = bars + 13;
  uint64_t* s_full = bars + 17;
  uint64_t* p_ready = bars + 18;      // (count 128)
  uint64_t* o_done = bars + 19;
  uint64_t* s_free = bars + 20;       // (count 128): the score row of a step is in registers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 22);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = warp_idx_uniform();
  const int lane = threadIdx.x & 31;

  // heavy (late) query tiles first; heads of one KV group adjacent for L2 reuse of K/V
  const int n_qt = p.S / FA1_BLK;
  const int head = blockIdx.x % p.Hq;
  const int rest = blockIdx.x / p.Hq;
  const int b = rest % p.batch;
  const int qt = n_qt - 1 - rest / p.batch;
  const int grp = head / p.g;
  const int q_col = (grp * (p.g + 2) + head % p.g) * D;
  const int k_col = (grp * (p.g + 2) + p.g) * D;
  const int v_col = k_col + D;
  const int row_base = b * p.S;
  const int nk = qt + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KS; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_ready, 128);
    mbar_init(o_done, 1);
    mbar_init(s_free, 128);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tm_qkv);
    prefetch_tmap(&tm_out);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base;          // 128 columns
  const uint32_t tmem_O = tmem_base + 128;    // D
  const uint32_t tmem_P = C::P_OVER_S ? tmem_base : tmem_base + 192;   // 64 (packed bf16 pairs)

  if (warp < 4) {
  reg_dealloc<56>();   // the softmax warpgroup takes these registers (whole warpgroups only)
  if (warp == 0) {
    // ---------------- producer: lanes [0, NBOX) load Q and the K blocks, lanes [NBOX, 2 NBOX)
    // the V blocks, one 64-column box each ----------------
    if (lane < 2 * NBOX) {
      const int c = lane % NBOX;
      const bool is_v = lane >= NBOX;
      if (lane == 0) mbar_expect_tx(q_full, L::TILE);
      if (!is_v)
        tma_load_2d(smem + L::Q_OFF + c * 16384, &tm_qkv, q_full, q_col + c * 64,
                    row_base + qt * FA1_BLK);
      for (int j = 0; j < nk; ++j) {
        const int st = j % KS;
        if (!is_v) {
          mbar_wait(&k_empty[st], ((j / KS) & 1) ^ 1, abort_flag, p.status, FT_ERR_WAIT_EMPTY);
          if (c == 0) mbar_expect_tx(&k_full[st], L::TILE);
          tma_load_2d(smem + L::K_OFF + st * L::TILE + c * 16384, &tm_qkv, &k_full[st],
                      k_col + c * 64, row_base + j * FA1_BLK);
        } else {
          mbar_wait(&v_empty[st], ((j / VS) & 1) ^ 1, abort_flag, p.status, FT_ERR_WAIT_EMPTY);
          if (c == 0) mbar_expect_tx(&v_full[st], L::TILE);
          tma_load_2d(smem + L::V_OFF + st * L::TILE + c * 16384, &tm_qkv, &v_full[st],
                      v_col + c * 64, row_base + j * FA1_BLK);
        }
      }
      if (lane == 0 && *abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer: in-order chain S(0), [S(j+1), P V(j)]...; the whole warp runs
    // the loop and the waits, one elected lane issues ----------------
    const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
    const uint32_t idesc_o = make_idesc_bf16(128, D, 0, 1);
    const uint32_t sQ = smem_u32(smem + L::Q_OFF), sK = smem_u32(smem + L::K_OFF);
    const uint32_t sV = smem_u32(smem + L::V_OFF);
    constexpr uint32_t TL = L::TILE >> 4;
    const uint32_t qa = smem_desc_lo(sQ, 16), kK0 = smem_desc_lo(sK, 16);
    const uint32_t vMN0 = smem_desc_lo(sV, 16384);
    // K-major operand, reduction step kk (16 elements): + (kk/4)*16384 + (kk%4)*32 bytes (blocks
    // of 64 columns); MN-major operand, step kk (16 rows of 128 B): + kk*2048 bytes
#define FT_KOFF(kk) ((((kk) / 4) * 16384 + ((kk) % 4) * 32) >> 4)
    auto issue_S = [&](int j) {
      const uint32_t ka = kK0 + (j % KS) * TL;
      umma_ss_lo<0>(tmem_S, qa, ka, idesc_s);
#pragma unroll
      for (int kk = 1; kk < D / 16; ++kk)
        umma_ss_lo<1>(tmem_S, qa + FT_KOFF(kk), ka + FT_KOFF(kk), idesc_s);
      umma_commit(s_full);
      umma_commit(&k_empty[j % KS]);
    };
#undef FT_KOFF
    auto issue_PV = [&](int j) {
      const uint32_t va = vMN0 + (j % VS) * TL;
      umma_ts_lo_dyn(tmem_O, tmem_P, va, idesc_o, j > 0 ? 1u : 0u);
#pragma unroll
      for (int kk = 1; kk < 8; ++kk)   // 16 bf16 of a row = 8 TMEM columns per k-step
        umma_ts_lo<1>(tmem_O, tmem_P + kk * 8, va + ((kk * 2048) >> 4), idesc_o);
      umma_commit(o_done);
      umma_commit(&v_empty[j % VS]);
    };
    mbar_wait(q_full, 0, abort_flag, p.status, FT_ERR_WAIT_FULL);
    mbar_wait(&k_full[0], 0, abort_flag, p.status, FT_ERR_WAIT_FULL);
    tc_fence_after();
    if (elect_one_sync()) issue_S(0);
    __syncwarp();
    for (int j = 0; j < nk; ++j) {
      if constexpr (!C::P_OVER_S) {
        // S of step j+1 goes to the tensor pipe as soon as the softmax warpgroup holds the score
        // row of step j in registers, i.e. while it is still exponentiating it
        if (j + 1 < nk) {
          mbar_wait(s_free, j & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_EMPTY);
          mbar_wait(&k_full[(j + 1) % KS], ((j + 1) / KS) & 1, abort_flag, p.status, FT_ERR_WAIT_FULL);
          tc_fence_after();
          if (elect_one_sync()) issue_S(j + 1);
          __syncwarp();
        }
      }
      mbar_wait(&v_full[j % VS], (j / VS) & 1, abort_flag, p.status, FT_ERR_WAIT_FULL);
      mbar_wait(p_ready, j & 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
      tc_fence_after();
      if (elect_one_sync()) issue_PV(j);
      __syncwarp();
      if constexpr (C::P_OVER_S) {
        // P sits in the columns of S: the next score block goes out BEHIND the P V product
        // that reads it (one thread's products run in order)
        if (j + 1 < nk) {
          mbar_wait(&k_full[(j + 1) % KS], ((j + 1) / KS) & 1, abort_flag, p.status, FT_ERR_WAIT_FULL);
          tc_fence_after();
          if (elect_one_sync()) issue_S(j + 1);
          __syncwarp();
        }
      }
    }
  }
  } else {
    reg_alloc<200>();
    // ---------------- softmax warpgroup: thread r owns query row r (= TMEM lane r) ----------------
    const int r = (warp & 3) * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int q_row = qt * FA1_BLK + r;  // position inside the sequence
    // staging of the output tile: the Q buffer, which the tensor core has finished reading once
    // the last score block is in registers
    uint8_t* sO = smem + L::Q_OFF;
    float m_ref = -INFINITY, l = 0.f;
    const uint64_t sl2x2 = pack_f32x2(p.scale_log2, p.scale_log2);
    uint64_t lsum2 = pack_f32x2(0.f, 0.f);
    for (int j = 0; j < nk; ++j) {
      mbar_wait(s_full, j & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_FULL);
      tc_fence_after();
      alignas(8) uint32_t s[128];   // the whole score row
      tmem_ld32(tmem_S + lane_off, s);
      tmem_ld32(tmem_S + lane_off + 32, s + 32);
      tmem_ld32(tmem_S + lane_off + 64, s + 64);
      tmem_ld32(tmem_S + lane_off + 96, s + 96);
      tmem_ld_wait();
      tc_fence_before();
      if constexpr (!C::P_OVER_S) mbar_arrive(s_free);
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
          mbar_wait(o_done, (j - 1) & 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
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
            tmem_ld32(tmem_O + lane_off + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int k = 0; k < 32; ++k) o[k] = __float_as_uint(__uint_as_float(o[k]) * alpha);
            tmem_st32(tmem_O + lane_off + c * 32, o);
          }
          tmem_st_wait();
        }
      }
      const uint64_t negm2 = pack_f32x2(-m_ref, -m_ref);
      // one interleaved stream over 16 chunks of 8 columns: scale, exponential (one pair in four
      // by polynomial on the FMA pipe), row sum, bf16 packing; P is stored after the stream
      uint64_t* s2 = reinterpret_cast<uint64_t*>(s);
      uint64_t acc0 = pack_f32x2(0.f, 0.f), acc1 = acc0, acc2 = acc0, acc3 = acc0;
      uint32_t pk[64];
#pragma unroll
      for (int c = 0; c < 16; ++c) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int i = c * 4 + q;
          uint64_t t = fma_f32x2(s2[i], sl2x2, negm2);
          float e0, e1;
          if (q < C::POLY) {
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
          pk[i] = pack_bf16x2(e0, e1);
        }
      }
      lsum2 = add_f32x2(lsum2, add_f32x2(add_f32x2(acc0, acc1), add_f32x2(acc2, acc3)));
      if (j > 0 && !o_waited) {   // the previous P V product has finished reading the P columns
        mbar_wait(o_done, (j - 1) & 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
        tc_fence_after();
      }
      tmem_st32(tmem_P + lane_off, pk);
      tmem_st32(tmem_P + lane_off + 32, pk + 32);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(p_ready);
    }
    {
      float l0, l1;
      unpack_f32x2(lsum2, l0, l1);
      l = l0 + l1;
    }
    // ---------------- epilogue: O / l -> bf16 -> TMA store; LSE ----------------
    mbar_wait(o_done, (nk - 1) & 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
    tc_fence_after();
    const float inv_l = 1.f / l;
#pragma unroll 1
    for (int c = 0; c < D / 32; ++c) {
      uint32_t o[32];
      tmem_ld32(tmem_O + lane_off + c * 32, o);
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
    named_bar_sync(1, 128);
    if (warp == 4 && lane == 0) {
#pragma unroll
      for (int c = 0; c < NBOX; ++c)
        tma_store_2d(&tm_out, sO + c * 16384, head * D + c * 64, row_base + qt * FA1_BLK);
      tma_commit_group();
      tma_wait_group<0>();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

// Launch of the one-tile forward kernel. `tq`: qkv map with 128 x 64 boxes, `to`: output map
// with 128 x 64 boxes.
template <int D>
static int launch_fa_fwd1_t(const CUtensorMap& tq, const CUtensorMap& to, int S, int Hq, int g,
                            int n_groups, int batch, float scale_log2, float* lse, int* status,
                            cudaStream_t st) {
  using L = FaFwd1Smem<D>;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(fa_fwd1_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             L::TOTAL) != cudaSuccess)
      return -10;
    attr = true;
  }
  FaFwd1Params p;
  p.S = S; p.Hq = Hq; p.g = g; p.n_groups = n_groups; p.batch = batch;
  p.scale_log2 = scale_log2;
  p.lse = lse;
  p.status = status;
  const int grid = (S / FA1_BLK) * batch * Hq;
  fa_fwd1_kernel<D><<<grid, FA1_THREADS, L::TOTAL, st>>>(tq, to, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int launch_fa_fwd1(const CUtensorMap& tq, const CUtensorMap& to, int D, int S, int Hq, int g,
                   int n_groups, int batch, float scale_log2, float* lse, int* status,
                   cudaStream_t st) {
  if (D == 64)
    return launch_fa_fwd1_t<64>(tq, to, S, Hq, g, n_groups, batch, scale_log2, lse, status, st);
  return launch_fa_fwd1_t<128>(tq, to, S, Hq, g, n_groups, batch, scale_log2, lse, status, st);
}

}  // namespace ft
