// Memory-bound kernels of the transformer block, the loss and the optimizer, written for
// sm_100a with 16-byte accesses everywhere and fp32 internal math:
//   embedding gather / scatter-add, residual-add + RMSNorm forward, RMSNorm backward (+ residual
//   gradient add, + weight-gradient partials), rotary embedding in place on the interleaved
//   QKV buffer, SwiGLU forward / backward, fused cross-entropy forward+backward (also the
//   vocab-parallel three-phase form), fused AdamW over a flat shard with a segment table, and
//   sum-of-squares for the gradient norm.
// These replace the reference's Triton kernels
// (exports/train_engine_0.5B/src/training_engine_tensor/triton_kernels.py:39-1397 and
// exports/train_engine_8b/src/training_engine_tensor/kernels.py:144-2054).
#include "ptx.cuh"
#include "swiglu_math.cuh"

namespace ft {

struct alignas(16) bf16x8 {
  uint32_t v[4];
};

__device__ __forceinline__ void unpack8(const bf16x8& p, float* f) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = bf16_lo(p.v[i]);
    f[2 * i + 1] = bf16_hi(p.v[i]);
  }
}
__device__ __forceinline__ bf16x8 pack8(const float* f) {
  bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = pack_bf16x2(f[2 * i], f[2 * i + 1]);
  return p;
}
// Stops the compiler from keeping the unpacked fp32 copies of a packed vector alive across
// this point (it would rather spend 16 registers than unpack twice).
__device__ __forceinline__ void opaque(bf16x8& p) {
  asm volatile("" : "+r"(p.v[0]), "+r"(p.v[1]), "+r"(p.v[2]), "+r"(p.v[3]));
}
__device__ __forceinline__ float round_bf16(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}

// Sum over the TPR threads that share a row. TPR == 32: one warp; TPR == 128: the whole CTA.
template <int TPR>
__device__ __forceinline__ float row_sum(float v, float* red, int warp_in_cta) {
  v = warp_sum(v);
  if (TPR == 32) return v;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[warp_in_cta] = v;
  __syncthreads();
  return red[0] + red[1] + red[2] + red[3];
}

// ---------------------------------------------------------------------------------------
// embedding
// ---------------------------------------------------------------------------------------
__global__ void embedding_fwd_kernel(const int64_t* __restrict__ ids,
                                     const __nv_bfloat16* __restrict__ w,
                                     __nv_bfloat16* __restrict__ out, int T, int H, float scale,
                                     int vocab_start, int vocab_rows) {
  const int t = blockIdx.x;
  const long id = ids[t] - vocab_start;
  const bool live = id >= 0 && id < vocab_rows;
  const bf16x8* src = reinterpret_cast<const bf16x8*>(w + (live ? id : 0) * (long)H);
  bf16x8* dst = reinterpret_cast<bf16x8*>(out + (long)t * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    float f[8];
    if (live) {
      unpack8(src[i], f);
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] *= scale;
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] = 0.f;
    }
    dst[i] = pack8(f);
  }
}

__global__ void embedding_bwd_kernel(const int64_t* __restrict__ ids,
                                     const __nv_bfloat16* __restrict__ dy, float* __restrict__ dw,
                                     int T, int H, float scale, int vocab_start, int vocab_rows) {
  const int t = blockIdx.x;
  const long id = ids[t] - vocab_start;
  if (id < 0 || id >= vocab_rows) return;
  const bf16x8* src = reinterpret_cast<const bf16x8*>(dy + (long)t * H);
  float4* dst = reinterpret_cast<float4*>(dw + id * (long)H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    float f[8];
    unpack8(src[i], f);
    atomicAdd(dst + 2 * i, make_float4(f[0] * scale, f[1] * scale, f[2] * scale, f[3] * scale));
    atomicAdd(dst + 2 * i + 1,
              make_float4(f[4] * scale, f[5] * scale, f[6] * scale, f[7] * scale));
  }
}

// ---------------------------------------------------------------------------------------
// RMSNorm forward with optional residual add:
//   h = bf16(res + x) (written when res != nullptr), rstd = rsqrt(mean(h^2) + eps),
//   y = bf16(h * rstd * w)
// NV = 16-byte vectors per thread, TPR = threads per row.
// ---------------------------------------------------------------------------------------
template <int NV, int TPR>
__global__ void __launch_bounds__(128)
add_rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ res, const __nv_bfloat16* __restrict__ x,
                       const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ h_out,
                       __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out, int T, int H,
                       float eps) {
  __shared__ float red[4];
  constexpr int ROWS_PER_CTA = 128 / TPR;
  const int sub = threadIdx.x / TPR;
  const int tr = threadIdx.x % TPR;
  const int warp = threadIdx.x >> 5;
  const bf16x8* wv = reinterpret_cast<const bf16x8*>(w);
  for (long row0 = (long)blockIdx.x * ROWS_PER_CTA; row0 < T; row0 += (long)gridDim.x * ROWS_PER_CTA) {
    const long row = row0 + sub;
    const bool live = row < T;
    const long r = live ? row : (T - 1);
    const bf16x8* xv = reinterpret_cast<const bf16x8*>(x + r * H);
    const bf16x8* rv = res ? reinterpret_cast<const bf16x8*>(res + r * H) : nullptr;
    float hf[NV][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      unpack8(xv[tr + i * TPR], hf[i]);
      if (rv) {
        float rf[8];
        unpack8(rv[tr + i * TPR], rf);
#pragma unroll
        for (int k = 0; k < 8; ++k) hf[i][k] = round_bf16(hf[i][k] + rf[k]);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) ss += hf[i][k] * hf[i][k];
    }
    ss = row_sum<TPR>(ss, red, warp);
    const float rstd = rsqrtf(ss / (float)H + eps);
    if (live) {
      if (tr == 0) rstd_out[row] = rstd;
      bf16x8* yv = reinterpret_cast<bf16x8*>(y + row * H);
      bf16x8* hv = (rv && h_out) ? reinterpret_cast<bf16x8*>(h_out + row * H) : nullptr;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        if (hv) hv[tr + i * TPR] = pack8(hf[i]);
        float wf[8], o[8];
        unpack8(wv[tr + i * TPR], wf);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = hf[i][k] * rstd * wf[k];
        yv[tr + i * TPR] = pack8(o);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// RMSNorm backward: dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres), written to dx_out
// (may alias dres); per-CTA weight-gradient partials sum_rows dy * xhat go to
// dw_partial[gridDim.x][H] and are folded by colsum_partials_kernel.
// ---------------------------------------------------------------------------------------
#ifndef FT_NORM_BWD_CPS
#define FT_NORM_BWD_CPS 3   // resident CTAs per SM the backward kernel is sized for
#endif
template <int NV, int TPR>
__global__ void __launch_bounds__(128, FT_NORM_BWD_CPS)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                   const __nv_bfloat16* dres, __nv_bfloat16* dx_out,
                   float* __restrict__ dw_partial, int T, int H) {
  __shared__ float red[4];
  extern __shared__ float dw_smem[];  // [H] when TPR == 32 (cross-warp fold), unused otherwise
  constexpr int ROWS_PER_CTA = 128 / TPR;
  const int sub = threadIdx.x / TPR;
  const int tr = threadIdx.x % TPR;
  const int warp = threadIdx.x >> 5;
  const bf16x8* wv = reinterpret_cast<const bf16x8*>(w);
  bf16x8 wp[NV];        // weights stay packed: they are unpacked where they are used
  float acc[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    wp[i] = wv[tr + i * TPR];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[i][k] = 0.f;
  }
  for (long row0 = (long)blockIdx.x * ROWS_PER_CTA; row0 < T; row0 += (long)gridDim.x * ROWS_PER_CTA) {
    const long row = row0 + sub;
    const bool live = row < T;
    const long r = live ? row : (T - 1);
    const bf16x8* dyv = reinterpret_cast<const bf16x8*>(dy + r * H);
    const bf16x8* hv = reinterpret_cast<const bf16x8*>(h + r * H);
    const bf16x8* rv = (dres && live) ? reinterpret_cast<const bf16x8*>(dres + row * H) : nullptr;
    // issue every load of the row first (packed, 4 registers per 8 values) ...
    bf16x8 dp[NV], hp[NV], rp[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      dp[i] = dyv[tr + i * TPR];
      hp[i] = hv[tr + i * TPR];
      if (rv) rp[i] = rv[tr + i * TPR];
    }
    const float rstd = rstd_in[r];
    // ... then pass 1: c = mean(dy * w * xhat), weight-gradient partials
    float c = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float d[8], hh[8], wf[8];
      unpack8(dp[i], d);
      unpack8(hp[i], hh);
      unpack8(wp[i], wf);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float xh = hh[k] * rstd;
        c += d[k] * wf[k] * xh;
        if (live) acc[i][k] += d[k] * xh;
      }
    }
    c = row_sum<TPR>(c, red, warp) / (float)H;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      opaque(dp[i]);
      opaque(hp[i]);
      opaque(wp[i]);
    }
    // pass 2: dx = rstd * (dy*w - xhat*c) (+ dres), recomputed from the packed registers
    if (live) {
      bf16x8* ov = reinterpret_cast<bf16x8*>(dx_out + row * H);
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        float d[8], hh[8], wf[8], o[8];
        unpack8(dp[i], d);
        unpack8(hp[i], hh);
        unpack8(wp[i], wf);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = rstd * (d[k] * wf[k] - hh[k] * rstd * c);
        if (rv) {
          float rf[8];
          unpack8(rp[i], rf);
#pragma unroll
          for (int k = 0; k < 8; ++k) o[k] += rf[k];
        }
        ov[tr + i * TPR] = pack8(o);
      }
    }
  }
  // fold the per-thread partials of this CTA into one [H] row
  float* outp = dw_partial + (long)blockIdx.x * H;
  if (TPR == 128) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float4* o4 = reinterpret_cast<float4*>(outp + (tr + i * TPR) * 8);
      o4[0] = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
      o4[1] = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
    }
  } else {
    for (int i = threadIdx.x; i < H; i += 128) dw_smem[i] = 0.f;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
      for (int k = 0; k < 8; ++k) atomicAdd(&dw_smem[(tr + i * TPR) * 8 + k], acc[i][k]);
    __syncthreads();
    for (int i = threadIdx.x; i < H; i += 128) outp[i] = dw_smem[i];
  }
}

// out[c] (=|+=) sum_p partial[p][c]. One CTA per 32 columns; COLSUM_GROUPS row-groups of 32 lanes
// each walk the partial rows with stride COLSUM_GROUPS (a handful of independent loads per
// thread: the kernel is pure latency) and are folded through shared memory in a fixed order.
constexpr int COLSUM_GROUPS = 32;
__global__ void __launch_bounds__(32 * COLSUM_GROUPS)
colsum_partials_kernel(const float* __restrict__ partial, float* __restrict__ out, int P, int H,
                       int accumulate) {
  __shared__ float red[COLSUM_GROUPS][33];
  const int cx = threadIdx.x & 31, px = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float s0 = 0.f, s1 = 0.f;
  if (c < H) {
    int p = px;
    for (; p + COLSUM_GROUPS < P; p += 2 * COLSUM_GROUPS) {
      s0 += partial[(long)p * H + c];
      s1 += partial[(long)(p + COLSUM_GROUPS) * H + c];
    }
    if (p < P) s0 += partial[(long)p * H + c];
  }
  red[px][cx] = s0 + s1;
  __syncthreads();
  if (px == 0 && c < H) {
    float s = red[0][cx];
#pragma unroll
    for (int k = 1; k < COLSUM_GROUPS; ++k) s += red[k][cx];
    out[c] = accumulate ? out[c] + s : s;
  }
}

// ---------------------------------------------------------------------------------------
// RoPE (rotate-half) in place on the q and k heads of the interleaved qkv buffer
// [T][n_groups * (g + 2) * D]. One thread rotates 8 + 8 elements (first / second half).
// pos = position_ids[t] when given, else t % S. inverse: transposed rotation (backward).
// ---------------------------------------------------------------------------------------
__global__ void rope_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t,
                            const int* __restrict__ position_ids, long T, int S, int n_groups,
                            int g, int D, int ld, int inverse) {
  const int half = D / 2;
  const int vec_per_head = half / 8;
  const int rot_heads = n_groups * (g + 1);
  const long total = T * rot_heads * vec_per_head;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long)gridDim.x * blockDim.x) {
    const int v = idx % vec_per_head;
    const long r1 = idx / vec_per_head;
    const int hd = r1 % rot_heads;
    const long t = r1 / rot_heads;
    const int grp = hd / (g + 1), in = hd % (g + 1);
    const int col = (grp * (g + 2) + in) * D + v * 8;
    const int pos = position_ids ? position_ids[t] : (int)(t % S);
    bf16x8* p1 = reinterpret_cast<bf16x8*>(qkv + t * ld + col);
    bf16x8* p2 = reinterpret_cast<bf16x8*>(qkv + t * ld + col + half);
    float x1[8], x2[8], o1[8], o2[8];
    unpack8(*p1, x1);
    unpack8(*p2, x2);
    const float4* c4 = reinterpret_cast<const float4*>(cos_t + (long)pos * half + v * 8);
    const float4* s4 = reinterpret_cast<const float4*>(sin_t + (long)pos * half + v * 8);
    float c[8], s[8];
    *reinterpret_cast<float4*>(c) = c4[0];
    *reinterpret_cast<float4*>(c + 4) = c4[1];
    *reinterpret_cast<float4*>(s) = s4[0];
    *reinterpret_cast<float4*>(s + 4) = s4[1];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float sn = inverse ? -s[k] : s[k];
      o1[k] = x1[k] * c[k] - x2[k] * sn;
      o2[k] = x2[k] * c[k] + x1[k] * sn;
    }
    *p1 = pack8(o1);
    *p2 = pack8(o2);
  }
}

// ---------------------------------------------------------------------------------------
// SwiGLU. y1 = [gate | up] per row (row length 2F), act = silu(gate) * up.
// ---------------------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ y1,
                                  __nv_bfloat16* __restrict__ act, long T, int F, int ld_y1,
                                  int ld_act) {
  const int vpr = F / 8;
  const long total = T * vpr;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long)gridDim.x * blockDim.x) {
    const long t = idx / vpr;
    const int v = idx % vpr;
    float gt[8], up[8], o[8];
    unpack8(*reinterpret_cast<const bf16x8*>(y1 + t * ld_y1 + v * 8), gt);
    unpack8(*reinterpret_cast<const bf16x8*>(y1 + t * ld_y1 + F + v * 8), up);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float sig = 1.f / (1.f + __expf(-gt[k]));
      o[k] = gt[k] * sig * up[k];
    }
    *reinterpret_cast<bf16x8*>(act + t * ld_act + v * 8) = pack8(o);
  }
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dact,
                                  const __nv_bfloat16* __restrict__ y1,
                                  __nv_bfloat16* __restrict__ dy1, long T, int F, int ld_dact,
                                  int ld_y1) {
  const int vpr = F / 8;
  const long total = T * vpr;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long)gridDim.x * blockDim.x) {
    const long t = idx / vpr;
    const int v = idx % vpr;
    float gt[8], up[8], d[8], dg[8], du[8];
    unpack8(*reinterpret_cast<const bf16x8*>(y1 + t * ld_y1 + v * 8), gt);
    unpack8(*reinterpret_cast<const bf16x8*>(y1 + t * ld_y1 + F + v * 8), up);
    unpack8(*reinterpret_cast<const bf16x8*>(dact + t * ld_dact + v * 8), d);
#pragma unroll
    for (int k = 0; k < 8; ++k) swiglu_bwd_elem(d[k], gt[k], up[k], dg[k], du[k]);
    *reinterpret_cast<bf16x8*>(dy1 + t * ld_y1 + v * 8) = pack8(dg);
    *reinterpret_cast<bf16x8*>(dy1 + t * ld_y1 + F + v * 8) = pack8(du);
  }
}

// ---------------------------------------------------------------------------------------
// Cross-entropy. One CTA per row, two passes over the row (the second one is served from L2):
//   pass 1: online (max, sum-exp) + target logit        -> stats[3][T] (max, sumexp, target)
//   pass 2: dlogits = (exp(l - gmax)/gsum - onehot) * mask/valid * loss_scale, in place
// Single-GPU use runs both phases in one launch (phase = 3). The vocab-parallel form runs
// phase 1, lets the tensor-parallel ranks combine the statistics, then runs phase 2 with the
// combined (gmax, gsum) per row.
// ---------------------------------------------------------------------------------------
constexpr int CE_THREADS = 512;

__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
  const float nm = fmaxf(m, m2);
  const float a = (m == -INFINITY) ? 0.f : __expf(m - nm);   // empty partials carry (-inf, 0)
  const float b = (m2 == -INFINITY) ? 0.f : __expf(m2 - nm);
  s = s * a + s2 * b;
  m = nm;
}

__global__ void __launch_bounds__(CE_THREADS)
cross_entropy_kernel(__nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ labels,
                     const float* __restrict__ mask, const float* __restrict__ valid_ptr,
                     float* __restrict__ stats, float* __restrict__ row_loss, int T, int V,
                     long ld, int vocab_start, float loss_scale, int phase) {
  __shared__ float sm[CE_THREADS / 32], ss[CE_THREADS / 32];
  __shared__ float bc[2];
  const int row = blockIdx.x;
  __nv_bfloat16* lrow = logits + (long)row * ld;
  const int nvec = V / 8;
  const int tail0 = nvec * 8;
  float gmax, gsum;
  const long lab = labels[row] - vocab_start;
  const bool lab_here = lab >= 0 && lab < V;
  if (phase & 1) {
    float m = -INFINITY, s = 0.f;
    for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
      float f[8];
      unpack8(reinterpret_cast<const bf16x8*>(lrow)[i], f);
      float lm = f[0];
#pragma unroll
      for (int k = 1; k < 8; ++k) lm = fmaxf(lm, f[k]);
      const float nm = fmaxf(m, lm);
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) acc += __expf(f[k] - nm);
      s = s * __expf(m - nm) + acc;
      m = nm;
    }
    for (int i = tail0 + threadIdx.x; i < V; i += CE_THREADS) {
      const float f = __bfloat162float(lrow[i]);
      online_merge(m, s, f, 1.f);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
      const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
      online_merge(m, s, m2, s2);
    }
    if ((threadIdx.x & 31) == 0) {
      sm[threadIdx.x >> 5] = m;
      ss[threadIdx.x >> 5] = s;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float M = sm[0], S = ss[0];
      for (int i = 1; i < CE_THREADS / 32; ++i) online_merge(M, S, sm[i], ss[i]);
      const float tgt = lab_here ? __bfloat162float(lrow[lab]) : 0.f;
      bc[0] = M;
      bc[1] = S;
      if (stats) {
        stats[row] = M;
        stats[T + row] = S;
        stats[2 * T + row] = tgt;
      }
      if (phase == 3 && row_loss) {
        const float mk = mask ? mask[row] : 1.f;
        row_loss[row] = (logf(S) + M - tgt) * mk;
      }
    }
    __syncthreads();
    gmax = bc[0];
    gsum = bc[1];
  } else {
    gmax = stats[row];
    gsum = stats[T + row];
  }
  if (!(phase & 2)) return;
  const float mk = mask ? mask[row] : 1.f;
  const float coef = mk / fmaxf(valid_ptr ? valid_ptr[0] : (float)T, 1.f) * loss_scale;
  const float inv = coef / gsum;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    float f[8];
    bf16x8* p = reinterpret_cast<bf16x8*>(lrow) + i;
    unpack8(*p, f);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = __expf(f[k] - gmax) * inv;
    if (lab_here && (lab >> 3) == i) f[lab & 7] -= coef;
    *p = pack8(f);
  }
  for (int i = tail0 + threadIdx.x; i < V; i += CE_THREADS) {
    float f = __expf(__bfloat162float(lrow[i]) - gmax) * inv;
    if (lab_here && lab == i) f -= coef;
    lrow[i] = __float2bfloat16_rn(f);
  }
}

// Vocab-parallel phase between the two: given the combined statistics (gmax[T], gsum[T],
// gtarget[T]) compute the masked per-row loss.
__global__ void ce_row_loss_kernel(const float* __restrict__ stats, const float* __restrict__ mask,
                                   float* __restrict__ row_loss, int T) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T) return;
  const float mk = mask ? mask[i] : 1.f;
  row_loss[i] = (logf(stats[T + i]) + stats[i] - stats[2 * T + i]) * mk;
}

// out[0] (=|+=) scale * sum(x[0..n)) / max(valid, 1); deterministic single-CTA tree.
__global__ void __launch_bounds__(1024)
reduce_sum_kernel(const float* __restrict__ x, long n, const float* __restrict__ valid_ptr,
                  float scale, float* __restrict__ out, int accumulate) {
  __shared__ float red[32];
  float s = 0.f;
  for (long i = threadIdx.x; i < n; i += blockDim.x) s += x[i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    s = warp_sum(s);
    if (threadIdx.x == 0) {
      const float d = valid_ptr ? fmaxf(valid_ptr[0], 1.f) : 1.f;
      const float r = s * scale / d;
      out[0] = accumulate ? out[0] + r : r;
    }
  }
}

// ---------------------------------------------------------------------------------------
// AdamW over a flat fp32 shard with per-segment (weight decay, lr multiplier).
// hyper[] lives in device memory so the launch can sit in a CUDA graph:
//   hyper = {lr, beta1, beta2, eps, bias_corr1, bias_corr2, clip, unused}
// seg_end[s] = exclusive end offset of segment s (ascending), seg_wd[s], seg_lr_mult[s].
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ p32, float* __restrict__ m, float* __restrict__ v,
             const float* __restrict__ g, __nv_bfloat16* __restrict__ p_bf16, long n,
             const float* __restrict__ hyper, const long* __restrict__ seg_end,
             const float* __restrict__ seg_wd, const float* __restrict__ seg_lr_mult, int nseg) {
  const float lr = hyper[0], b1 = hyper[1], b2 = hyper[2], eps = hyper[3];
  const float inv_bc1 = 1.f / hyper[4], inv_bc2 = 1.f / hyper[5], clip = hyper[6];
  const long nvec = n / 4;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long)gridDim.x * blockDim.x) {
    const long e0 = i * 4;
    // segment of the first element (binary search), then walk
    int lo = 0, hi = nseg - 1;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (seg_end[mid] > e0) hi = mid; else lo = mid + 1;
    }
    int seg = lo;
    float4 p4 = reinterpret_cast<float4*>(p32)[i];
    float4 m4 = reinterpret_cast<float4*>(m)[i];
    float4 v4 = reinterpret_cast<float4*>(v)[i];
    const float4 g4 = reinterpret_cast<const float4*>(g)[i];
    float pp[4] = {p4.x, p4.y, p4.z, p4.w}, mm[4] = {m4.x, m4.y, m4.z, m4.w};
    float vv[4] = {v4.x, v4.y, v4.z, v4.w}, gg[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      while (seg < nseg - 1 && seg_end[seg] <= e0 + k) ++seg;
      const float wd = seg_wd[seg], lrm = seg_lr_mult[seg];
      const float gr = gg[k] * clip;
      mm[k] = b1 * mm[k] + (1.f - b1) * gr;
      vv[k] = b2 * vv[k] + (1.f - b2) * gr * gr;
      const float upd = (mm[k] * inv_bc1) / (sqrtf(vv[k] * inv_bc2) + eps) + wd * pp[k];
      pp[k] -= lr * lrm * upd;
    }
    reinterpret_cast<float4*>(p32)[i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (p_bf16) {
      uint2 o;
      o.x = pack_bf16x2(pp[0], pp[1]);
      o.y = pack_bf16x2(pp[2], pp[3]);
      reinterpret_cast<uint2*>(p_bf16)[i] = o;
    }
  }
}

// out[0] += sum(x^2) (fp32 atomics over per-CTA partials; callers zero out[0] first)
__global__ void __launch_bounds__(256)
sumsq_kernel(const float* __restrict__ x, long n, float* __restrict__ out) {
  __shared__ float red[8];
  float s = 0.f;
  const long nvec = n / 4;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long)gridDim.x * blockDim.x) {
    const float4 a = reinterpret_cast<const float4*>(x)[i];
    s += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
  }
  if (blockIdx.x == 0)
    for (long i = nvec * 4 + threadIdx.x; i < n; i += blockDim.x) s += x[i] * x[i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 8) {
    s = red[threadIdx.x];
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) s += __shfl_xor_sync(0xffu, s, o);
    if (threadIdx.x == 0) atomicAdd(out, s);
  }
}

// clip[0] = min(1, max_norm / (sqrt(sumsq[0]) + 1e-6)); norm_out[0] = sqrt(sumsq[0])
__global__ void clip_coef_kernel(const float* __restrict__ sumsq, float max_norm,
                                 float* __restrict__ hyper_clip, float* __restrict__ norm_out) {
  const float nrm = sqrtf(sumsq[0]);
  norm_out[0] = nrm;
  hyper_clip[0] = max_norm > 0.f ? fminf(1.f, max_norm / (nrm + 1e-6f)) : 1.f;
}

// One thread: advance the device-resident optimizer step counter and derive this step's
// scalars, so that a replayed CUDA graph needs nothing from the host.
//   sched = [max_lr, min_lr, warmup_iters, lr_decay_iters, wsd_decay_iters, beta1, beta2, eps]
//   hyper[0..5] = lr, beta1, beta2, eps, 1 - beta1^t, 1 - beta2^t   (t = step after increment)
// The learning rate is the warmup - stable - decay schedule evaluated at the step count
// before the increment.
__global__ void adam_hyper_kernel(int* __restrict__ step, const float* __restrict__ sched,
                                  float* __restrict__ hyper) {
  const int it = step[0];
  const double max_lr = sched[0], min_lr = sched[1];
  const int warmup = (int)sched[2], decay = (int)sched[3], wsd = (int)sched[4];
  double lr;
  if (warmup > 0 && it < warmup) {
    lr = max_lr * it / warmup;
  } else if (wsd <= 0) {
    lr = it <= decay ? max_lr : min_lr;
  } else {
    const int stable_end = decay - wsd;
    if (it <= stable_end) lr = max_lr;
    else if (it > decay) lr = min_lr;
    else lr = min_lr + (2.0 * pow(0.5, (double)(it - stable_end) / wsd) - 1.0) * (max_lr - min_lr);
  }
  const int t = it + 1;
  step[0] = t;
  const double b1 = sched[5], b2 = sched[6];
  hyper[0] = (float)lr;
  hyper[1] = sched[5];
  hyper[2] = sched[6];
  hyper[3] = sched[7];
  hyper[4] = (float)(1.0 - pow(b1, (double)t));
  hyper[5] = (float)(1.0 - pow(b2, (double)t));
}

static int grid_for(long work_items, int threads, int cap_mult = 8) {
  long b = (work_items + threads - 1) / threads;
  const long cap = 148L * cap_mult;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (int)b;
}

}  // namespace ft

using namespace ft;
#define FT_LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? 0 : -100)

extern "C" int ft_embedding_fwd(const void* ids, const void* w, void* out, int T, int H,
                                float scale, int vocab_start, int vocab_rows,
                                cudaStream_t st) {
  if (H % 8) return -1;
  embedding_fwd_kernel<<<T, 128, 0, st>>>((const int64_t*)ids, (const __nv_bfloat16*)w,
                                          (__nv_bfloat16*)out, T, H, scale, vocab_start,
                                          vocab_rows);
  return FT_LAUNCH_OK();
}

extern "C" int ft_embedding_bwd(const void* ids, const void* dy, void* dw, int T, int H,
                                float scale, int vocab_start, int vocab_rows,
                                cudaStream_t st) {
  if (H % 8) return -1;
  embedding_bwd_kernel<<<T, 128, 0, st>>>((const int64_t*)ids, (const __nv_bfloat16*)dy,
                                          (float*)dw, T, H, scale, vocab_start, vocab_rows);
  return FT_LAUNCH_OK();
}

// Picks (NV, TPR) such that H == NV * TPR * 8. Returns 0 when the shape is unsupported.
static int norm_cfg(int H, int* nv, int* tpr) {
  const int t = (H <= 1024) ? 32 : 128;
  if (H % (t * 8)) return 0;
  const int n = H / (t * 8);
  if (n != 1 && n != 2 && n != 4 && n != 8) return 0;
  *nv = n;
  *tpr = t;
  return 1;
}

#define FT_NORM_DISPATCH(NVV, TPRV, CALL)                                     \
  if (nv == NVV && tpr == TPRV) { constexpr int NV = NVV; constexpr int TPR = TPRV; CALL; }

extern "C" int ft_add_rmsnorm_fwd(const void* res, const void* x, const void* w, void* h_out,
                                  void* y, void* rstd, int T, int H, float eps,
                                  cudaStream_t st) {
  int nv, tpr;
  if (!norm_cfg(H, &nv, &tpr)) return -1;
  const int rows_per_cta = 128 / tpr;
  const int grid = grid_for((long)(T + rows_per_cta - 1) / rows_per_cta, 1, 16);
#define CALL_FWD                                                                          \
  add_rmsnorm_fwd_kernel<NV, TPR><<<grid, 128, 0, st>>>(                                  \
      (const __nv_bfloat16*)res, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w,        \
      (__nv_bfloat16*)h_out, (__nv_bfloat16*)y, (float*)rstd, T, H, eps)
  FT_NORM_DISPATCH(1, 32, CALL_FWD)
  FT_NORM_DISPATCH(2, 32, CALL_FWD)
  FT_NORM_DISPATCH(4, 32, CALL_FWD)
  FT_NORM_DISPATCH(2, 128, CALL_FWD)
  FT_NORM_DISPATCH(4, 128, CALL_FWD)
  FT_NORM_DISPATCH(8, 128, CALL_FWD)
#undef CALL_FWD
  return FT_LAUNCH_OK();
}

// Number of CTAs (= rows of dw_partial) the backward kernel will use for T rows of width H.
extern "C" int ft_rmsnorm_bwd_partials(int T, int H) {
  int nv, tpr;
  if (!norm_cfg(H, &nv, &tpr)) return -1;
  const int rows_per_cta = 128 / tpr;
  return grid_for((long)(T + rows_per_cta - 1) / rows_per_cta, 1, FT_NORM_BWD_CPS);
}

extern "C" int ft_rmsnorm_bwd(const void* dy, const void* h, const void* w, const void* rstd,
                              const void* dres, void* dx_out, void* dw_partial, void* dw,
                              int accumulate, int T, int H, cudaStream_t st) {
  int nv, tpr;
  if (!norm_cfg(H, &nv, &tpr)) return -1;
  const int grid = ft_rmsnorm_bwd_partials(T, H);
  const size_t smem = tpr == 32 ? (size_t)H * 4 : 0;
#define CALL_BWD                                                                          \
  rmsnorm_bwd_kernel<NV, TPR><<<grid, 128, smem, st>>>(                                   \
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)h, (const __nv_bfloat16*)w,         \
      (const float*)rstd, (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx_out,             \
      (float*)dw_partial, T, H)
  FT_NORM_DISPATCH(1, 32, CALL_BWD)
  FT_NORM_DISPATCH(2, 32, CALL_BWD)
  FT_NORM_DISPATCH(4, 32, CALL_BWD)
  FT_NORM_DISPATCH(2, 128, CALL_BWD)
  FT_NORM_DISPATCH(4, 128, CALL_BWD)
  FT_NORM_DISPATCH(8, 128, CALL_BWD)
#undef CALL_BWD
  if (cudaGetLastError() != cudaSuccess) return -100;
  colsum_partials_kernel<<<(H + 31) / 32, 32 * COLSUM_GROUPS, 0, st>>>((const float*)dw_partial, (float*)dw,
                                                        grid, H, accumulate);
  return FT_LAUNCH_OK();
}

extern "C" int ft_rope(void* qkv, const void* cos_t, const void* sin_t, const void* position_ids,
                       long T, int S, int n_groups, int g, int D, int ld, int inverse,
                       cudaStream_t st) {
  if (D % 16 || ld % 8) return -1;
  const long total = T * n_groups * (g + 1) * (D / 16);
  rope_kernel<<<grid_for(total, 256, 16), 256, 0, st>>>((__nv_bfloat16*)qkv, (const float*)cos_t,
                                                        (const float*)sin_t,
                                                        (const int*)position_ids, T, S, n_groups,
                                                        g, D, ld, inverse);
  return FT_LAUNCH_OK();
}

extern "C" int ft_swiglu_fwd(const void* y1, void* act, long T, int F, int ld_y1, int ld_act,
                             cudaStream_t st) {
  if (F % 8 || ld_y1 % 8 || ld_act % 8) return -1;
  swiglu_fwd_kernel<<<grid_for(T * (F / 8), 256, 16), 256, 0, st>>>(
      (const __nv_bfloat16*)y1, (__nv_bfloat16*)act, T, F, ld_y1, ld_act);
  return FT_LAUNCH_OK();
}

extern "C" int ft_swiglu_bwd(const void* dact, const void* y1, void* dy1, long T, int F,
                             int ld_dact, int ld_y1, cudaStream_t st) {
  if (F % 8 || ld_y1 % 8 || ld_dact % 8) return -1;
  swiglu_bwd_kernel<<<grid_for(T * (F / 8), 256, 16), 256, 0, st>>>(
      (const __nv_bfloat16*)dact, (const __nv_bfloat16*)y1, (__nv_bfloat16*)dy1, T, F, ld_dact,
      ld_y1);
  return FT_LAUNCH_OK();
}

// phase: 1 = statistics only, 2 = gradient only (stats hold the combined values),
// 3 = both in one launch (single-GPU). Rows must be 16-byte aligned (ld % 8 == 0).
extern "C" int ft_cross_entropy(void* logits, const void* labels, const void* mask,
                                const void* valid, void* stats, void* row_loss, int T, int V,
                                long ld, int vocab_start, float loss_scale, int phase,
                                cudaStream_t st) {
  if (ld % 8) return -1;
  cross_entropy_kernel<<<T, CE_THREADS, 0, st>>>((__nv_bfloat16*)logits, (const int64_t*)labels,
                                                 (const float*)mask, (const float*)valid,
                                                 (float*)stats, (float*)row_loss, T, V, ld,
                                                 vocab_start, loss_scale, phase);
  return FT_LAUNCH_OK();
}

extern "C" int ft_ce_row_loss(const void* stats, const void* mask, void* row_loss, int T,
                              cudaStream_t st) {
  ce_row_loss_kernel<<<(T + 255) / 256, 256, 0, st>>>((const float*)stats, (const float*)mask,
                                                      (float*)row_loss, T);
  return FT_LAUNCH_OK();
}

extern "C" int ft_reduce_sum(const void* x, long n, const void* valid, float scale, void* out,
                             int accumulate, cudaStream_t st) {
  reduce_sum_kernel<<<1, 1024, 0, st>>>((const float*)x, n, (const float*)valid, scale,
                                        (float*)out, accumulate);
  return FT_LAUNCH_OK();
}

extern "C" int ft_adamw(void* p32, void* m, void* v, const void* g, void* p_bf16, long n,
                        const void* hyper, const void* seg_end, const void* seg_wd,
                        const void* seg_lr_mult, int nseg, cudaStream_t st) {
  if (n % 4) return -1;
  adamw_kernel<<<grid_for(n / 4, 256, 16), 256, 0, st>>>(
      (float*)p32, (float*)m, (float*)v, (const float*)g, (__nv_bfloat16*)p_bf16, n,
      (const float*)hyper, (const long*)seg_end, (const float*)seg_wd, (const float*)seg_lr_mult,
      nseg);
  return FT_LAUNCH_OK();
}

extern "C" int ft_sumsq(const void* x, long n, void* out, cudaStream_t st) {
  sumsq_kernel<<<grid_for(n / 4 + 1, 256, 8), 256, 0, st>>>((const float*)x, n, (float*)out);
  return FT_LAUNCH_OK();
}

extern "C" int ft_clip_coef(const void* sumsq, float max_norm, void* hyper_clip, void* norm_out,
                            cudaStream_t st) {
  clip_coef_kernel<<<1, 1, 0, st>>>((const float*)sumsq, max_norm, (float*)hyper_clip,
                                    (float*)norm_out);
  return FT_LAUNCH_OK();
}

extern "C" int ft_adam_hyper(void* step, const void* sched, void* hyper, cudaStream_t st) {
  adam_hyper_kernel<<<1, 1, 0, st>>>((int*)step, (const float*)sched, (float*)hyper);
  return FT_LAUNCH_OK();
}

// ---------------------------------------------------------------------------------------
// Allocation-free variant of ft_rmsnorm_bwd (declared and documented in ft_noalloc.h).
// The weight-gradient partials go to a scratch array that is part of the library image.
// ---------------------------------------------------------------------------------------
#include "ft_noalloc.h"

static __device__ __align__(256) float g_noalloc_dw_partial[FT_NOALLOC_MAX_PARTIALS * FT_NOALLOC_MAX_HIDDEN];

// In host code the symbol above is only a handle; the kernels need its device address, which
// is looked up once per device (with that device current) and cached here.
static float* g_noalloc_ptr[64] = {nullptr};

static float* noalloc_scratch() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!g_noalloc_ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_dw_partial) != cudaSuccess || !p) return nullptr;
    g_noalloc_ptr[dev] = static_cast<float*>(p);
  }
  return g_noalloc_ptr[dev];
}

extern "C" int ft_rmsnorm_bwd_noalloc(const void* dy, const void* h, const void* w,
                                      const void* rstd, const void* dres, void* dx_out, void* dw,
                                      int accumulate, int T, int H, cudaStream_t st) {
  if (H > FT_NOALLOC_MAX_HIDDEN) return -2;
  int nv, tpr;
  if (!norm_cfg(H, &nv, &tpr)) return -1;
  float* scratch = noalloc_scratch();
  if (!scratch) return -3;
  const int rows_per_cta = 128 / tpr;
  long want = (static_cast<long>(T) + rows_per_cta - 1) / rows_per_cta;
  const int grid = want < 1 ? 1 : (want > FT_NOALLOC_MAX_PARTIALS ? FT_NOALLOC_MAX_PARTIALS : (int)want);
  const size_t smem = tpr == 32 ? (size_t)H * 4 : 0;
#define CALL_BWD_NA                                                                       \
  rmsnorm_bwd_kernel<NV, TPR><<<grid, 128, smem, st>>>(                                   \
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)h, (const __nv_bfloat16*)w,         \
      (const float*)rstd, (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx_out, scratch, T, H)
  FT_NORM_DISPATCH(1, 32, CALL_BWD_NA)
  FT_NORM_DISPATCH(2, 32, CALL_BWD_NA)
  FT_NORM_DISPATCH(4, 32, CALL_BWD_NA)
  FT_NORM_DISPATCH(2, 128, CALL_BWD_NA)
  FT_NORM_DISPATCH(4, 128, CALL_BWD_NA)
  FT_NORM_DISPATCH(8, 128, CALL_BWD_NA)
#undef CALL_BWD_NA
  if (cudaGetLastError() != cudaSuccess) return -100;
  colsum_partials_kernel<<<(H + 31) / 32, 32 * COLSUM_GROUPS, 0, st>>>(scratch, (float*)dw, grid, H, accumulate);
  return FT_LAUNCH_OK();
}
