// The gated unit of the experts' first products, in the forms the designs use:
//   g' = min(g, limit), u' = clamp(u, -limit, limit);  out = g' * sigmoid(alpha g') * (u' + up_shift)
// limit = +inf, alpha = 1 and up_shift = 0 give silu(g) * u; a finite limit, alpha = 1.702 and up_shift = 1 the clamped
// unit.  All in fp32.
#pragma once
#include <math.h>

__device__ __forceinline__ float nhv_glu(float g, float u, float limit, float alpha, float up_shift) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.0f + expf(-alpha * g)) * (u + up_shift);
}
