// Causal GQA FlashAttention forward for sm_100a (head_dim 64 or 128), reading q/k/v straight out
// of the interleaved projection buffer qkv[T][n_groups*(g+2)*D] through strided TMA boxes and
// writing out[T][Hq*D] plus the log-sum-exp.
//
// One CTA owns two consecutive 128-row query tiles of one (batch, head) and ping-pongs them:
//   warp 0      TMA producer  (Q once, then K_j / V_j rings)
//   warp 1      MMA issuer    (tcgen05.mma: S_w = Q_w K_j^T, O_w += P_w V_j; TMEM accumulators)
//   warps 4-7   softmax of tile 0 (one thread per query row, no shuffles)
//   warps 8-11  softmax of tile 1
// While one warpgroup exponentiates, the tensor core works for the other tile. The running
// maximum is only refreshed when it grew by more than 2^8 ("lazy rescale"), which keeps the
// TMEM round-trip of O off the common path. P goes through shared memory in the 128-byte
// swizzled K-major layout the MMA reads.
//
// Replaces the reference's Hopper FlashAttention forward kernels
// (ops/attention/flash_attn_dsl/flash_fwd.py:31-660, src/flash_attn_dsl/flash_fwd.py:1-803).
#include "ptx.cuh"
#include "tma_host.h"

namespace ft {

int get_tmap_2d(CUtensorMap* out, const void* base, int elt, uint64_t rows, uint64_t cols,
                uint64_t ld, uint32_t box_r, uint32_t box_c);

constexpr int FA_THREADS = 384;
constexpr int FA_BLK = 128;
#ifndef FA_POLY
#define FA_POLY 1   // pairs out of every 4 whose 2^x is evaluated by polynomial
#endif

struct FaFwdParams {
  int S, Hq, g, n_groups, batch;
  float scale_log2;  // softmax scale * log2(e)
  float* lse;        // [B][Hq][S]
  int* status;
};

template <int D, int KS, int VS>
struct FaFwdSmem {
  static constexpr int TILE = FA_BLK * D * 2;        // one 128 x D bf16 tile
  static constexpr int Q_OFF = 0;                    // 2 tiles
  static constexpr int K_OFF = 2 * TILE;
  static constexpr int V_OFF = K_OFF + KS * TILE;
  static constexpr int P_OFF = V_OFF + VS * TILE;    // 2 x (128 x 128 bf16)
  static constexpr int BAR_OFF = P_OFF + 2 * 32768;
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
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // KS (<=2)
  uint64_t* k_empty = bars + 3;
  uint64_t* v_full = bars + 5;
  uint64_t* v_empty = bars + 7;
  uint64_t* s_full = bars + 9;        // 2
  uint64_t* p_ready = bars + 11;      // 2
  uint64_t* o_done = bars + 13;       // 2
  uint64_t* s_free = bars + 15;       // 2 (count 128): the score row of a step is in registers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
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
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
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

  if (warp < 4) {
  reg_dealloc<96>();   // TMA / MMA warps need few registers, the softmax warps a whole score row
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
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer ----------------
      const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_o = make_idesc_bf16(128, D, 0, 1);
      const uint32_t sQ = smem_u32(smem + L::Q_OFF), sK = smem_u32(smem + L::K_OFF);
      const uint32_t sV = smem_u32(smem + L::V_OFF), sP = smem_u32(smem + L::P_OFF);
      // descriptor low words: K-major step kk: +(kk/4)*16384 + (kk%4)*32 bytes; MN-major: + kk*2048
      const uint32_t qK0 = smem_desc_lo(sQ, 16), kK0 = smem_desc_lo(sK, 16);
      const uint32_t pK0 = smem_desc_lo(sP, 16), vMN0 = smem_desc_lo(sV, 16384);
      constexpr uint32_t TL = L::TILE >> 4, PB = 32768 >> 4;
#define FT_KOFF(kk) ((((kk) / 4) * 16384 + ((kk) % 4) * 32) >> 4)
#define FT_MNOFF(kk) (((kk) * 2048) >> 4)
      auto issue_S = [&](int w, int j) {
        const uint32_t qa = qK0 + w * TL, ka = kK0 + (j % KS) * TL;
        umma_ss_lo<0>(tmem_S[w], qa, ka, idesc_s);
#pragma unroll
        for (int kk = 1; kk < D / 16; ++kk)
          umma_ss_lo<1>(tmem_S[w], qa + FT_KOFF(kk), ka + FT_KOFF(kk), idesc_s);
        umma_commit(&s_full[w]);
      };
      auto issue_PV = [&](int w, int j) {
        const uint32_t pa = pK0 + w * PB, va = vMN0 + (j % VS) * TL;
        umma_ss_lo_dyn(tmem_O[w], pa, va, idesc_o, j > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 1; kk < 8; ++kk)
          umma_ss_lo<1>(tmem_O[w], pa + FT_KOFF(kk), va + FT_MNOFF(kk), idesc_o);
        umma_commit(&o_done[w]);
      };
      mbar_wait(q_full, 0, abort_flag, p.status, FT_ERR_WAIT_FULL);
      mbar_wait(&k_full[0], 0, abort_flag, p.status, FT_ERR_WAIT_FULL);
      tc_fence_after();
      issue_S(0, 0);
      issue_S(1, 0);
      umma_commit(&k_empty[0]);
      for (int j = 0; j < n_total; ++j) {
        const int vs = j % VS;
        // S of step j+1 goes to the tensor pipe as soon as the softmax warpgroup holds the
        // score row of step j in registers, i.e. while it is still exponentiating it.
        bool next_k_ready = false;
        for (int w = 0; w < 2; ++w) {
          if (j + 1 >= n_kv[w]) continue;
          mbar_wait(&s_free[w], j & 1, abort_flag, p.status, FT_ERR_WAIT_TMEM_EMPTY);
          if (!next_k_ready) {
            mbar_wait(&k_full[(j + 1) % KS], ((j + 1) / KS) & 1, abort_flag, p.status,
                      FT_ERR_WAIT_FULL);
            next_k_ready = true;
          }
          tc_fence_after();
          issue_S(w, j + 1);
          if (w == 1) umma_commit(&k_empty[(j + 1) % KS]);
        }
        mbar_wait(&v_full[vs], (j / VS) & 1, abort_flag, p.status, FT_ERR_WAIT_FULL);
        for (int w = 0; w < 2; ++w) {
          if (j >= n_kv[w]) continue;
          mbar_wait(&p_ready[w], j & 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
          tc_fence_after();
          issue_PV(w, j);
          if (w == 1) umma_commit(&v_empty[vs]);
        }
      }
    }
  }
#undef FT_KOFF
#undef FT_MNOFF
  } else {
    reg_alloc<200>();
    // ---------------- softmax warpgroups ----------------
    const int w = (warp - 4) >> 2;           // query tile of this warpgroup
    const int r = threadIdx.x - 128 - w * 128;  // row inside the tile == TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int qt = 2 * pair + w;
    const int q_row = qt * FA_BLK + r;  // position inside the sequence
    uint8_t* sP = smem + L::P_OFF + w * 32768;
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
      float mx0 = __uint_as_float(s[0]), mx1 = __uint_as_float(s[1]);
#pragma unroll
      for (int k = 2; k < 128; k += 4) {
        mx0 = max3(mx0, __uint_as_float(s[k]), __uint_as_float(s[k + 1]));
        if (k + 3 < 128) mx1 = max3(mx1, __uint_as_float(s[k + 2]), __uint_as_float(s[k + 3]));
      }
      const float mx = fmaxf(mx0, mx1);
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
      // staged so that each stage is a long run of independent instructions
      uint64_t* s2 = reinterpret_cast<uint64_t*>(s);
#pragma unroll
      for (int i = 0; i < 64; ++i) s2[i] = fma_f32x2(s2[i], sl2x2, negm2);
      // FA_POLY of every 4 pairs take the polynomial path: the transcendental unit is the
      // scarce pipe of this loop (8 cycles per warp instruction), the FMA pipe has room.
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        if ((i & 3) < FA_POLY) {
          s2[i] = exp2_poly_f32x2(s2[i]);
        } else {
          s[2 * i] = __float_as_uint(fast_exp2(__uint_as_float(s[2 * i])));
          s[2 * i + 1] = __float_as_uint(fast_exp2(__uint_as_float(s[2 * i + 1])));
        }
      }
      uint64_t acc0 = s2[0], acc1 = s2[1], acc2 = s2[2], acc3 = s2[3];
#pragma unroll
      for (int i = 4; i < 64; i += 4) {
        acc0 = add_f32x2(acc0, s2[i]);
        acc1 = add_f32x2(acc1, s2[i + 1]);
        acc2 = add_f32x2(acc2, s2[i + 2]);
        acc3 = add_f32x2(acc3, s2[i + 3]);
      }
      lsum2 = add_f32x2(lsum2, add_f32x2(add_f32x2(acc0, acc1), add_f32x2(acc2, acc3)));
      if (j > 0 && !o_waited) {   // the P buffer is still read by the previous P V product
        mbar_wait(&o_done[w], (j - 1) & 1, abort_flag, p.status, FT_ERR_WAIT_MISC);
        tc_fence_after();
      }
#pragma unroll
      for (int c = 0; c < 16; ++c) {  // 16 chunks of 8 columns = one 16-byte store each
        uint4 u;
        u.x = pack_bf16x2_int(__uint_as_float(s[c * 8 + 0]), __uint_as_float(s[c * 8 + 1]));
        u.y = pack_bf16x2_int(__uint_as_float(s[c * 8 + 2]), __uint_as_float(s[c * 8 + 3]));
        u.z = pack_bf16x2_int(__uint_as_float(s[c * 8 + 4]), __uint_as_float(s[c * 8 + 5]));
        u.w = pack_bf16x2_int(__uint_as_float(s[c * 8 + 6]), __uint_as_float(s[c * 8 + 7]));
        uint8_t* rowp = sP + (c >> 3) * 16384 + r * 128;
        *reinterpret_cast<uint4*>(rowp + (((c & 7) ^ (r & 7)) << 4)) = u;
      }
      tc_fence_before();
      fence_proxy_async_smem();
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
      uint8_t* rowp = sP + (c >> 1) * 16384 + r * 128;
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
        tma_store_2d(&tm_out, sP + c * 16384, head * D + c * 64, row_base + qt * FA_BLK);
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
  if (D == 64) return launch_fa_fwd<64, 2, 2>(tq, to, p, st);
  return launch_fa_fwd<128, 1, 1>(tq, to, p, st);
}
