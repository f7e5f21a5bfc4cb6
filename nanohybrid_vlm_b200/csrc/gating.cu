// Small elementwise steps around gated sub-blocks, all computed in fp32 and rounded once:
//
//   sigmoid_mul     out[t, c] = x[t, c] * sigmoid(g[t, c])          (an output gate before the output projection)
//   add_row_bias    x[t, c] += bias[c], in place                     (the bias of a projection whose product has none)
//   clamped_glu     out[t, c] = g' * sigmoid(alpha * g') * (u' + 1), g' = min(gate, limit), u' = clamp(up, -limit, limit)
//                   for gate_up [T, 2 I] with the gate in the first half of each row
//
// Each takes eight columns per thread where the width and the row strides are multiples of 8 and the pointers lie
// on 16-byte boundaries, else one.
#include <math.h>

#include "nhv_common.cuh"
#include "nhv_vec8.cuh"

static inline int gating_blocks(size_t items) {
  const size_t b = (items + 255) / 256;
  return (int)(b < (size_t)1 << 20 ? b : (size_t)1 << 20);
}
static inline bool aligned16(const void* p) { return ((uintptr_t)p % 16) == 0; }

__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }

template <typename T, int VEC>
__global__ void sigmoid_mul_kernel(T* out, int out_stride, const T* x, int x_stride,      // out may be x itself
                                   const T* __restrict__ g, int g_stride, int width, size_t total) {
  pdl_prologue();
  for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC; i < total; i += (size_t)gridDim.x * blockDim.x * VEC) {
    const size_t t = i / width;
    const int c = (int)(i - t * width);
    if constexpr (VEC == 8) {
      float xv[8], gv[8];
      nhv_load8(xv, x + t * x_stride + c);
      nhv_load8(gv, g + t * g_stride + c);
#pragma unroll
      for (int e = 0; e < 8; ++e) xv[e] *= sigmoid_f(gv[e]);
      nhv_store8(out + t * out_stride + c, xv);
    } else {
      out[t * out_stride + c] = from_f32<T>(to_f32<T>(x[t * x_stride + c]) * sigmoid_f(to_f32<T>(g[t * g_stride + c])));
    }
  }
}

NHV_API int nhv_sigmoid_mul(int dtype, void* out, int out_stride, const void* x, int x_stride, const void* g, int g_stride,
                            int n_rows, int width, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NHV_REQUIRE(n_rows > 0 && width > 0, "sigmoid_mul: bad sizes");
  const size_t total = (size_t)n_rows * width;
  const bool vec = width % 8 == 0 && out_stride % 8 == 0 && x_stride % 8 == 0 && g_stride % 8 == 0 && aligned16(out) &&
                   aligned16(x) && aligned16(g);
#define GO(T, V)                                                                                                     \
  nhv_launch(sigmoid_mul_kernel<T, V>, gating_blocks(total / V), 256, 0, stream, (T*)out, out_stride, (const T*)x, x_stride, \
             (const T*)g, g_stride, width, total)
  if (dtype == NHV_F32) { if (vec) GO(float, 8); else GO(float, 1); }
  else if (dtype == NHV_BF16) { if (vec) GO(__nv_bfloat16, 8); else GO(__nv_bfloat16, 1); }
  else NHV_REQUIRE(false, "sigmoid_mul: unknown dtype %d", dtype);
#undef GO
  NHV_CHECK_LAUNCH("sigmoid_mul");
  return 0;
}

template <typename T, int VEC>
__global__ void add_row_bias_kernel(T* __restrict__ x, const T* __restrict__ bias, int width, size_t total) {
  pdl_prologue();
  for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC; i < total; i += (size_t)gridDim.x * blockDim.x * VEC) {
    const int c = (int)(i % width);
    if constexpr (VEC == 8) {
      float xv[8], bv[8];
      nhv_load8(xv, x + i);
      nhv_load8(bv, bias + c);
#pragma unroll
      for (int e = 0; e < 8; ++e) xv[e] += bv[e];
      nhv_store8(x + i, xv);
    } else {
      x[i] = from_f32<T>(to_f32<T>(x[i]) + to_f32<T>(bias[c]));
    }
  }
}

NHV_API int nhv_add_row_bias(int dtype, void* x, const void* bias, int n_rows, int width, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NHV_REQUIRE(n_rows > 0 && width > 0, "add_row_bias: bad sizes");
  const size_t total = (size_t)n_rows * width;
  const bool vec = width % 8 == 0 && aligned16(x) && aligned16(bias);
#define GO(T, V) nhv_launch(add_row_bias_kernel<T, V>, gating_blocks(total / V), 256, 0, stream, (T*)x, (const T*)bias, width, total)
  if (dtype == NHV_F32) { if (vec) GO(float, 8); else GO(float, 1); }
  else if (dtype == NHV_BF16) { if (vec) GO(__nv_bfloat16, 8); else GO(__nv_bfloat16, 1); }
  else NHV_REQUIRE(false, "add_row_bias: unknown dtype %d", dtype);
#undef GO
  NHV_CHECK_LAUNCH("add_row_bias");
  return 0;
}

__device__ __forceinline__ float clamped_glu(float g, float u, float limit, float alpha) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
}

template <typename T, int VEC>
__global__ void clamped_glu_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int inter, size_t total, float limit,
                                   float alpha) {
  pdl_prologue();
  for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC; i < total; i += (size_t)gridDim.x * blockDim.x * VEC) {
    const size_t t = i / inter;
    const int c = (int)(i - t * inter);
    const T* row = gate_up + t * 2 * inter;
    if constexpr (VEC == 8) {
      float gv[8], uv[8];
      nhv_load8(gv, row + c);
      nhv_load8(uv, row + inter + c);
#pragma unroll
      for (int e = 0; e < 8; ++e) gv[e] = clamped_glu(gv[e], uv[e], limit, alpha);
      nhv_store8(out + i, gv);
    } else {
      out[i] = from_f32<T>(clamped_glu(to_f32<T>(row[c]), to_f32<T>(row[inter + c]), limit, alpha));
    }
  }
}

NHV_API int nhv_clamped_glu(int dtype, void* out, const void* gate_up, int n_rows, int inter, float limit, float alpha,
                            cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NHV_REQUIRE(n_rows > 0 && inter > 0, "clamped_glu: bad sizes");
  const size_t total = (size_t)n_rows * inter;
  const bool vec = inter % 8 == 0 && aligned16(out) && aligned16(gate_up);
#define GO(T, V)                                                                                                   \
  nhv_launch(clamped_glu_kernel<T, V>, gating_blocks(total / V), 256, 0, stream, (T*)out, (const T*)gate_up, inter, total, \
             limit, alpha)
  if (dtype == NHV_F32) { if (vec) GO(float, 8); else GO(float, 1); }
  else if (dtype == NHV_BF16) { if (vec) GO(__nv_bfloat16, 8); else GO(__nv_bfloat16, 1); }
  else NHV_REQUIRE(false, "clamped_glu: unknown dtype %d", dtype);
#undef GO
  NHV_CHECK_LAUNCH("clamped_glu");
  return 0;
}

// out[t, c] = x[t, c] * sigmoid(g[t, c / group]): one gate per head of `group` columns.  out may be x itself.
// x_head: the distance between two heads in a row of x (group where the heads are packed; more where each head is
// padded, as the output of attention over padded heads is).
template <typename T>
__global__ void sigmoid_mul_heads_kernel(T* out, int out_stride, const T* x, int x_stride, const T* __restrict__ g,
                                         int g_stride, int width, int group, int x_head, size_t total) {
  pdl_prologue();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / width;
    const int c = (int)(i - t * width);
    const int h = c / group;
    out[t * out_stride + c] = from_f32<T>(to_f32<T>(x[t * x_stride + (size_t)h * x_head + (c - h * group)]) *
                                          sigmoid_f(to_f32<T>(g[t * g_stride + h])));
  }
}

NHV_API int nhv_sigmoid_mul_heads(int dtype, void* out, int out_stride, const void* x, int x_stride, const void* g,
                                  int g_stride, int n_rows, int width, int group, int x_head, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NHV_REQUIRE(n_rows > 0 && width > 0 && group > 0 && width % group == 0 && x_head >= group,
              "sigmoid_mul_heads: %d columns do not divide into heads of %d", width, group);
  const size_t total = (size_t)n_rows * width;
  if (dtype == NHV_F32)
    nhv_launch(sigmoid_mul_heads_kernel<float>, gating_blocks(total), 256, 0, stream, (float*)out, out_stride, (const float*)x,
               x_stride, (const float*)g, g_stride, width, group, x_head, total);
  else if (dtype == NHV_BF16)
    nhv_launch(sigmoid_mul_heads_kernel<__nv_bfloat16>, gating_blocks(total), 256, 0, stream, (__nv_bfloat16*)out, out_stride,
               (const __nv_bfloat16*)x, x_stride, (const __nv_bfloat16*)g, g_stride, width, group, x_head, total);
  else
    NHV_REQUIRE(false, "sigmoid_mul_heads: unknown dtype %d", dtype);
  NHV_CHECK_LAUNCH("sigmoid_mul_heads");
  return 0;
}

// x = max(x, 0)^2 in place, computed in fp32 and rounded once (the unit of a feed-forward without a gate).
template <typename T, int VEC>
__global__ void relu_squared_kernel(T* __restrict__ x, size_t total) {
  pdl_prologue();
  for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC; i < total; i += (size_t)gridDim.x * blockDim.x * VEC) {
    if constexpr (VEC == 8) {
      float v[8];
      nhv_load8(v, x + i);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float p = fmaxf(v[e], 0.f);
        v[e] = p * p;
      }
      nhv_store8(x + i, v);
    } else {
      const float p = fmaxf(to_f32<T>(x[i]), 0.f);
      x[i] = from_f32<T>(p * p);
    }
  }
}

NHV_API int nhv_relu_squared(int dtype, void* x, size_t total, cudaStream_t stream) {
  if (total == 0) return 0;
  const bool vec = total % 8 == 0 && aligned16(x);
#define GO(T, V) nhv_launch(relu_squared_kernel<T, V>, gating_blocks(total / V), 256, 0, stream, (T*)x, total)
  if (dtype == NHV_F32) { if (vec) GO(float, 8); else GO(float, 1); }
  else if (dtype == NHV_BF16) { if (vec) GO(__nv_bfloat16, 8); else GO(__nv_bfloat16, 1); }
  else NHV_REQUIRE(false, "relu_squared: unknown dtype %d", dtype);
#undef GO
  NHV_CHECK_LAUNCH("relu_squared");
  return 0;
}

// x = gelu_tanh(x) in place, gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))), computed in fp32 and rounded
// once (the unit of a feed-forward without a gate).
__device__ __forceinline__ float gating_gelu_tanh(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T, int VEC>
__global__ void gelu_tanh_kernel(T* __restrict__ x, size_t total) {
  pdl_prologue();
  for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC; i < total; i += (size_t)gridDim.x * blockDim.x * VEC) {
    if constexpr (VEC == 8) {
      float v[8];
      nhv_load8(v, x + i);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = gating_gelu_tanh(v[e]);
      nhv_store8(x + i, v);
    } else {
      x[i] = from_f32<T>(gating_gelu_tanh(to_f32<T>(x[i])));
    }
  }
}

NHV_API int nhv_gelu_tanh(int dtype, void* x, size_t total, cudaStream_t stream) {
  if (total == 0) return 0;
  const bool vec = total % 8 == 0 && aligned16(x);
#define GO(T, V) nhv_launch(gelu_tanh_kernel<T, V>, gating_blocks(total / V), 256, 0, stream, (T*)x, total)
  if (dtype == NHV_F32) { if (vec) GO(float, 8); else GO(float, 1); }
  else if (dtype == NHV_BF16) { if (vec) GO(__nv_bfloat16, 8); else GO(__nv_bfloat16, 1); }
  else NHV_REQUIRE(false, "gelu_tanh: unknown dtype %d", dtype);
#undef GO
  NHV_CHECK_LAUNCH("gelu_tanh");
  return 0;
}

// Logits in place (fp32): z <- z * scale, then, with cap > 0, z <- cap * tanh(z / cap).
__global__ void scale_softcap_kernel(float* __restrict__ z, float scale, float cap, size_t total) {
  pdl_prologue();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const float v = z[i] * scale;
    z[i] = cap > 0.f ? cap * tanhf(v / cap) : v;
  }
}

NHV_API int nhv_scale_softcap(float* z, float scale, float cap, size_t total, cudaStream_t stream) {
  if (total == 0) return 0;
  nhv_launch(scale_softcap_kernel, gating_blocks(total), 256, 0, stream, z, scale, cap, total);
  NHV_CHECK_LAUNCH("scale_softcap");
  return 0;
}
