// The Adam element update shared by the multi-tensor optimizer kernel and the
// fused dense reduce-scatter + AdamW + all-gather kernel. Files that include
// this must be compiled without fast-math and with -fmad=false so that each
// operation rounds separately, in the order of the PyTorch reference.
#pragma once

namespace sga {

struct AdamScalars {
  float beta1, omb1, beta2, omb2, bc1, bc2, eps;
};

// Returns the update (wd * w + u); m, v are advanced in place.
__device__ __forceinline__ float adam_update(float w, float g, float& m, float& v, float wd, int adams,
                                             const AdamScalars& s, float* u_out = nullptr) {
  const float m0 = m, v0 = v;
  const float m1 = m0 * s.beta1 + g * s.omb1;
  const float g2 = (g * s.omb2) * g;
  float v1, mh, vh;
  if (adams) {
    v1 = (m0 * m0) * s.beta2 + g2;
    mh = m1;
    vh = v1;
  } else {
    v1 = v0 * s.beta2 + g2;
    mh = m1 / s.bc1;
    vh = v1 / s.bc2;
  }
  const float u = mh / (sqrtf(vh) + s.eps);
  m = m1;
  v = v1;
  if (u_out) *u_out = u;
  return wd * w + u;
}

}  // namespace sga
