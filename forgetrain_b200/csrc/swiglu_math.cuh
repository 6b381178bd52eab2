// Arithmetic of the SwiGLU backward, shared by the stand-alone kernel (elementwise.cu) and the
// FC2-dgrad GEMM epilogue (gemm_sm100.cu) so that both give bitwise the same result.
#pragma once

namespace ft {

// act = silu(g) * u;  d g = d * sig * (1 + g (1 - sig)) * u;  d u = d * g * sig
__device__ __forceinline__ void swiglu_bwd_elem(float d, float g, float u, float& dg, float& du) {
  const float sig = __fdividef(1.f, 1.f + __expf(-g));
  dg = d * sig * (1.f + g * (1.f - sig)) * u;
  du = d * g * sig;
}

}  // namespace ft
