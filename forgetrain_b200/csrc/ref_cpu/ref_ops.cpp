// Host C++ statement of every device op (fp32 arrays, OpenMP over rows), independent of both
// the CUDA kernels and the PyTorch oracle. It is the third leg of the numerics checks: the
// CPU test-suite compares it with the PyTorch oracle, the GPU test-suite compares the CUDA
// kernels with it. All tensors are dense row-major float arrays; `round_bf16 != 0` applies
// the storage rounding (round-to-nearest-even to bfloat16) at the points where the device
// kernels write bf16.
//
// Op semantics follow the reference's baseline ops
// (exports/train_engine_0.5B/src/training_engine_tensor/kernels.py:39-56,265-335,
//  triton_kernels.py:39-178, 186-294, 302-406, 414-607, 645-791).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

namespace {

inline float bf16_round(float x) {
  uint32_t u;
  std::memcpy(&u, &x, 4);
  if ((u & 0x7f800000u) == 0x7f800000u) return x;  // inf / nan unchanged
  const uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  u &= 0xffff0000u;
  float y;
  std::memcpy(&y, &u, 4);
  return y;
}
inline float store(float x, int round_bf16) { return round_bf16 ? bf16_round(x) : x; }

}  // namespace

extern "C" {

// D[M,N] (=|+=) alpha * sum_k A(m,k) * B(n,k). a_mn / b_mn as in the device GEMM: 0 = the
// operand is stored [rows][ld] with k contiguous, 1 = stored [k][ld] with the row contiguous.
void ftref_gemm(const float* A, const float* B, float* D, int M, int N, int K, int lda, int ldb,
                int ldd, int a_mn, int b_mn, float alpha, int accumulate, int round_bf16) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    std::vector<double> acc(N, 0.0);
    for (int k = 0; k < K; ++k) {
      const double a = a_mn ? A[(size_t)k * lda + m] : A[(size_t)m * lda + k];
      if (b_mn) {
        const float* brow = B + (size_t)k * ldb;
        for (int n = 0; n < N; ++n) acc[n] += a * brow[n];
      } else {
        for (int n = 0; n < N; ++n) acc[n] += a * B[(size_t)n * ldb + k];
      }
    }
    for (int n = 0; n < N; ++n) {
      const float v = static_cast<float>(acc[n]) * alpha;
      float* d = D + (size_t)m * ldd + n;
      *d = accumulate ? *d + v : store(v, round_bf16);
    }
  }
}

void ftref_embedding_fwd(const int64_t* ids, const float* w, float* out, int T, int H,
                         float scale, int vocab_start, int vocab_rows, int round_bf16) {
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; ++t) {
    const int64_t r = ids[t] - vocab_start;
    for (int h = 0; h < H; ++h)
      out[(size_t)t * H + h] =
          (r >= 0 && r < vocab_rows) ? store(w[(size_t)r * H + h] * scale, round_bf16) : 0.f;
  }
}

void ftref_embedding_bwd(const int64_t* ids, const float* dy, float* dw, int T, int H,
                         float scale, int vocab_start, int vocab_rows) {
  for (int t = 0; t < T; ++t) {
    const int64_t r = ids[t] - vocab_start;
    if (r < 0 || r >= vocab_rows) continue;
    for (int h = 0; h < H; ++h) dw[(size_t)r * H + h] += scale * dy[(size_t)t * H + h];
  }
}

// h = round(res + x) (h = x when res == nullptr); y = h * rstd * w; rstd = rsqrt(mean(h^2)+eps)
void ftref_add_rmsnorm_fwd(const float* res, const float* x, const float* w, float* h, float* y,
                           float* rstd, int T, int H, float eps, int round_bf16) {
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; ++t) {
    double ss = 0.0;
    for (int j = 0; j < H; ++j) {
      const size_t i = (size_t)t * H + j;
      const float hv = res ? store(res[i] + x[i], round_bf16) : x[i];
      h[i] = hv;
      ss += (double)hv * hv;
    }
    const float r = 1.0f / std::sqrt(static_cast<float>(ss / H) + eps);
    rstd[t] = r;
    for (int j = 0; j < H; ++j) {
      const size_t i = (size_t)t * H + j;
      y[i] = store(h[i] * r * w[j], round_bf16);
    }
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres); dw (+)= sum_t dy * xhat
void ftref_rmsnorm_bwd(const float* dy, const float* h, const float* w, const float* rstd,
                       const float* dres, float* dx, float* dw, int accumulate, int T, int H,
                       int round_bf16) {
  std::vector<double> dwn(H, 0.0);
#pragma omp parallel
  {
    std::vector<double> local(H, 0.0);
#pragma omp for schedule(static)
    for (int t = 0; t < T; ++t) {
      const float r = rstd[t];
      double c = 0.0;
      for (int j = 0; j < H; ++j) {
        const size_t i = (size_t)t * H + j;
        c += (double)dy[i] * w[j] * (h[i] * r);
      }
      c /= H;
      for (int j = 0; j < H; ++j) {
        const size_t i = (size_t)t * H + j;
        const float xhat = h[i] * r;
        float v = r * (dy[i] * w[j] - xhat * static_cast<float>(c));
        if (dres) v += dres[i];
        dx[i] = store(v, round_bf16);
        local[j] += (double)dy[i] * xhat;
      }
    }
#pragma omp critical
    for (int j = 0; j < H; ++j) dwn[j] += local[j];
  }
  for (int j = 0; j < H; ++j) dw[j] = (accumulate ? dw[j] : 0.f) + static_cast<float>(dwn[j]);
}

// In-place rotate-half rotary embedding of the q heads and the k head of every KV group of
// qkv[T][G*(g+2)*D]; token t has position pos[t] (or t % S when pos == nullptr).
void ftref_rope(float* qkv, const float* cos_t, const float* sin_t, const int32_t* pos, int T,
                int S, int G, int g, int D, int inverse, int round_bf16) {
  const int half = D / 2;
  const int ld = G * (g + 2) * D;
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; ++t) {
    const int p = pos ? pos[t] : t % S;
    for (int grp = 0; grp < G; ++grp)
      for (int hd = 0; hd <= g; ++hd) {  // q heads, then k
        float* x = qkv + (size_t)t * ld + (size_t)(grp * (g + 2) + hd) * D;
        for (int j = 0; j < half; ++j) {
          const float c = cos_t[(size_t)p * half + j];
          const float s = inverse ? -sin_t[(size_t)p * half + j] : sin_t[(size_t)p * half + j];
          const float x1 = x[j], x2 = x[j + half];
          x[j] = store(x1 * c - x2 * s, round_bf16);
          x[j + half] = store(x2 * c + x1 * s, round_bf16);
        }
      }
  }
}

void ftref_swiglu_fwd(const float* y1, float* act, int T, int F, int round_bf16) {
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; ++t)
    for (int j = 0; j < F; ++j) {
      const float gate = y1[(size_t)t * 2 * F + j], up = y1[(size_t)t * 2 * F + F + j];
      act[(size_t)t * F + j] = store(gate / (1.f + std::exp(-gate)) * up, round_bf16);
    }
}

// FC1 with the activation folded in, the statement of the device kernel's fused epilogue: per
// row, gate_j = alpha * <a, w_j>, up_j = alpha * <a, w_{F+j}>, both stored (rounded) into Y, and
// act_j = silu(gate_j) * up_j computed FROM THE ROUNDED values, as the device epilogue does.
void ftref_linear_swiglu(const float* A, const float* W, float* Y, float* act, int M, int F, int K,
                         int lda, int ldw, float alpha, int round_bf16) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    const float* a = A + (size_t)m * lda;
    for (int j = 0; j < F; ++j) {
      double g = 0.0, u = 0.0;
      const float* wg = W + (size_t)j * ldw;
      const float* wu = W + (size_t)(F + j) * ldw;
      for (int k = 0; k < K; ++k) {
        g += (double)a[k] * wg[k];
        u += (double)a[k] * wu[k];
      }
      const float gate = store(static_cast<float>(g) * alpha, round_bf16);
      const float up = store(static_cast<float>(u) * alpha, round_bf16);
      Y[(size_t)m * 2 * F + j] = gate;
      Y[(size_t)m * 2 * F + F + j] = up;
      act[(size_t)m * F + j] = store(gate / (1.f + std::exp(-gate)) * up, round_bf16);
    }
  }
}

void ftref_swiglu_bwd(const float* dact, const float* y1, float* dy1, int T, int F,
                      int round_bf16) {
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; ++t)
    for (int j = 0; j < F; ++j) {
      const float gate = y1[(size_t)t * 2 * F + j], up = y1[(size_t)t * 2 * F + F + j];
      const float sig = 1.f / (1.f + std::exp(-gate));
      const float g = dact[(size_t)t * F + j];
      dy1[(size_t)t * 2 * F + j] = store(g * sig * (1.f + gate * (1.f - sig)) * up, round_bf16);
      dy1[(size_t)t * 2 * F + F + j] = store(g * gate * sig, round_bf16);
    }
}

// FC2 dgrad with the SwiGLU backward folded in, the statement of the device kernel's fused
// epilogue: per row, d act_j = alpha * <dy, w2[:, j]> is ROUNDED as the separate dgrad GEMM would
// store it and (d gate_j, d up_j) follow from it and the forward FC1 output; the [M][F] gradient of
// the activation is never materialised. W2 is stored [K][ldw] (K = hidden size, F columns).
void ftref_linear_dgrad_swiglu_bwd(const float* DY, const float* W2, const float* Y1, float* DY1,
                                   int M, int F, int K, int lddy, int ldw, float alpha,
                                   int round_bf16) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    const float* dy = DY + (size_t)m * lddy;
    for (int j = 0; j < F; ++j) {
      double a = 0.0;
      for (int k = 0; k < K; ++k) a += (double)dy[k] * W2[(size_t)k * ldw + j];
      const float g = store(static_cast<float>(a) * alpha, round_bf16);
      const float gate = Y1[(size_t)m * 2 * F + j], up = Y1[(size_t)m * 2 * F + F + j];
      const float sig = 1.f / (1.f + std::exp(-gate));
      DY1[(size_t)m * 2 * F + j] = store(g * sig * (1.f + gate * (1.f - sig)) * up, round_bf16);
      DY1[(size_t)m * 2 * F + F + j] = store(g * gate * sig, round_bf16);
    }
  }
}

// loss = sum(mask*ce)/valid (returned); dlogits = (softmax - onehot) * mask/valid * loss_scale.
// Labels outside [vocab_start, vocab_start+V) contribute no target logit (vocabulary shard).
float ftref_cross_entropy(const float* logits, const int64_t* labels, const float* mask,
                          float valid, float* dlogits, int T, int V, int vocab_start,
                          float loss_scale, int round_bf16) {
  double total = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : total)
  for (int t = 0; t < T; ++t) {
    const float* row = logits + (size_t)t * V;
    float mx = -std::numeric_limits<float>::infinity();
    for (int j = 0; j < V; ++j) mx = std::max(mx, row[j]);
    double se = 0.0;
    for (int j = 0; j < V; ++j) se += std::exp((double)row[j] - mx);
    const int64_t lab = labels[t] - vocab_start;
    const bool in = lab >= 0 && lab < V;
    const float tgt = in ? row[lab] : 0.f;
    const float m = mask ? mask[t] : 1.f;
    total += (std::log(se) + mx - tgt) * m;
    const float coef = m / valid * loss_scale;
    for (int j = 0; j < V; ++j) {
      float p = static_cast<float>(std::exp((double)row[j] - mx) / se);
      if (in && j == lab) p -= 1.f;
      dlogits[(size_t)t * V + j] = store(p * coef, round_bf16);
    }
  }
  return static_cast<float>(total / valid);
}

// Causal GQA attention over qkv[B*S][G*(g+2)*D] (per KV group: g query heads, k, v).
// out[B*S][G*g*D]; lse[B][G*g][S] (natural log).
void ftref_attention_fwd(const float* qkv, float* out, float* lse, int B, int S, int G, int g,
                         int D, float scale, int round_bf16) {
  const int ld = G * (g + 2) * D, Hq = G * g;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int b = 0; b < B; ++b)
    for (int hq = 0; hq < Hq; ++hq) {
      const int grp = hq / g, hd = hq % g;
      std::vector<double> s(S), acc(D);
      for (int i = 0; i < S; ++i) {
        const float* q = qkv + (size_t)(b * S + i) * ld + (size_t)(grp * (g + 2) + hd) * D;
        double mx = -1e300;
        for (int j = 0; j <= i; ++j) {
          const float* k = qkv + (size_t)(b * S + j) * ld + (size_t)(grp * (g + 2) + g) * D;
          double dot = 0.0;
          for (int d = 0; d < D; ++d) dot += (double)q[d] * k[d];
          s[j] = dot * scale;
          mx = std::max(mx, s[j]);
        }
        double se = 0.0;
        std::fill(acc.begin(), acc.end(), 0.0);
        for (int j = 0; j <= i; ++j) {
          const double p = std::exp(s[j] - mx);
          se += p;
          const float* v = qkv + (size_t)(b * S + j) * ld + (size_t)(grp * (g + 2) + g + 1) * D;
          for (int d = 0; d < D; ++d) acc[d] += p * v[d];
        }
        lse[((size_t)b * Hq + hq) * S + i] = static_cast<float>(mx + std::log(se));
        float* o = out + (size_t)(b * S + i) * Hq * D + (size_t)hq * D;
        for (int d = 0; d < D; ++d) o[d] = store(static_cast<float>(acc[d] / se), round_bf16);
      }
    }
}

// dqkv in the layout of qkv.
void ftref_attention_bwd(const float* dout, const float* qkv, const float* out, const float* lse,
                         float* dqkv, int B, int S, int G, int g, int D, float scale,
                         int round_bf16) {
  const int ld = G * (g + 2) * D, Hq = G * g;
  std::vector<double> acc((size_t)B * S * ld, 0.0);
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int b = 0; b < B; ++b)
    for (int grp = 0; grp < G; ++grp) {
      for (int hd = 0; hd < g; ++hd) {
        const int hq = grp * g + hd;
        for (int i = 0; i < S; ++i) {
          const size_t qoff = (size_t)(b * S + i) * ld + (size_t)(grp * (g + 2) + hd) * D;
          const float* q = qkv + qoff;
          const float* o = out + (size_t)(b * S + i) * Hq * D + (size_t)hq * D;
          const float* dO = dout + (size_t)(b * S + i) * Hq * D + (size_t)hq * D;
          double delta = 0.0;
          for (int d = 0; d < D; ++d) delta += (double)o[d] * dO[d];
          const double l = lse[((size_t)b * Hq + hq) * S + i];
          for (int j = 0; j <= i; ++j) {
            const size_t koff = (size_t)(b * S + j) * ld + (size_t)(grp * (g + 2) + g) * D;
            const size_t voff = koff + D;
            const float* k = qkv + koff;
            const float* v = qkv + voff;
            double dot = 0.0, dp = 0.0;
            for (int d = 0; d < D; ++d) {
              dot += (double)q[d] * k[d];
              dp += (double)dO[d] * v[d];
            }
            const double p = std::exp(dot * scale - l);
            const double ds = p * (dp - delta) * scale;
            for (int d = 0; d < D; ++d) {
              acc[voff + d] += p * dO[d];
              acc[qoff + d] += ds * k[d];
              acc[koff + d] += ds * q[d];
            }
          }
        }
      }
    }
  const size_t n = (size_t)B * S * ld;
  for (size_t i = 0; i < n; ++i) dqkv[i] = store(static_cast<float>(acc[i]), round_bf16);
}

// AdamW with decoupled weight decay and bias correction on fp32 master weights; p_out (may be
// null) receives the updated value in storage precision.
void ftref_adamw(float* p, float* m, float* v, const float* g, float* p_out, int64_t n, float lr,
                 float beta1, float beta2, float eps, float wd, int step, float clip,
                 int round_bf16) {
  const float bc1 = 1.f - std::pow(beta1, (float)step), bc2 = 1.f - std::pow(beta2, (float)step);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const float gg = g[i] * clip;
    m[i] = beta1 * m[i] + (1.f - beta1) * gg;
    v[i] = beta2 * v[i] + (1.f - beta2) * gg * gg;
    const float upd = (m[i] / bc1) / (std::sqrt(v[i] / bc2) + eps) + wd * p[i];
    p[i] -= lr * upd;
    if (p_out) p_out[i] = store(p[i], round_bf16);
  }
}

double ftref_sumsq(const float* x, int64_t n) {
  double s = 0.0;
#pragma omp parallel for reduction(+ : s) schedule(static)
  for (int64_t i = 0; i < n; ++i) s += (double)x[i] * x[i];
  return s;
}

}  // extern "C"
