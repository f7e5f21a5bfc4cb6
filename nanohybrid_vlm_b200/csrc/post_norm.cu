// A sub-block's output normed and added onto a residual stream kept in 32-bit floats (blocks that norm what a
// sub-block returns rather than what it reads).
//
//   postnorm_stream:  y = a                                       (one term without a norm of its own)
//                     y = ca * a / rms(a) * wa (+ cb * b / rms(b) * wb)   (terms that pass a norm of their own first)
//                     s = stream[t] + y / rms(y) * w * ls         (ls optional: a scale per channel)
//                     stream[t] = s;  rounded[t] = s in the storage type (optional: what the next sub-block reads)
//   stream_round:     rounded = stream in the storage type
//
// rms(v) = sqrt(mean(v^2) + eps).  Everything is computed in fp32; a, b and the weights are in the storage type.
// One block per row; the rows of a and b live in shared memory between the passes.
#include "nhv_common.cuh"

template <typename T>
__global__ void postnorm_stream_kernel(float* __restrict__ stream, T* __restrict__ rounded, const T* __restrict__ a,
                                       const T* __restrict__ wa, float ca, const T* __restrict__ b,
                                       const T* __restrict__ wb, float cb, const T* __restrict__ w,
                                       const T* __restrict__ ls, int width, float eps, float side_eps) {
  extern __shared__ float rowbuf[];
  __shared__ float red[33];
  pdl_prologue();
  float* ya = rowbuf;
  float* yb = rowbuf + width;
  const size_t at = (size_t)blockIdx.x * width;
  float sa = 0.f, sb = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float va = to_f32<T>(a[at + c]);
    ya[c] = va;
    sa = fmaf(va, va, sa);
    if (b) {
      const float vb = to_f32<T>(b[at + c]);
      yb[c] = vb;
      sb = fmaf(vb, vb, sb);
    }
  }
  float ra = 1.f, rb = 1.f;
  if (wa) ra = 1.0f / sqrtf(block_sum(sa, red) / (float)width + side_eps);
  if (b && wb) rb = 1.0f / sqrtf(block_sum(sb, red) / (float)width + side_eps);
  float sy = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float y = ya[c];
    if (wa) y = ca * (y * ra * to_f32<T>(wa[c]));
    else y *= ca;
    if (b) y += cb * (wb ? yb[c] * rb * to_f32<T>(wb[c]) : yb[c]);
    ya[c] = y;
    sy = fmaf(y, y, sy);
  }
  const float ry = 1.0f / sqrtf(block_sum(sy, red) / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = ya[c] * ry * to_f32<T>(w[c]);
    if (ls) v *= to_f32<T>(ls[c]);
    const float s = stream[at + c] + v;
    stream[at + c] = s;
    if (rounded) rounded[at + c] = from_f32<T>(s);
  }
}

NHV_API int nhv_postnorm_stream(int dtype, float* stream_rows, void* rounded, const void* a, const void* wa, float ca,
                                const void* b, const void* wb, float cb, const void* w, const void* ls, int n_rows,
                                int width, float eps, float side_eps, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NHV_REQUIRE(n_rows > 0 && width > 0 && stream_rows && a && w, "postnorm_stream: bad arguments");
  NHV_REQUIRE(b || !wb, "postnorm_stream: a second norm weight without a second term");
  const size_t smem = (size_t)2 * width * sizeof(float);
  NHV_REQUIRE(smem <= 200 * 1024, "postnorm_stream: width %d is beyond the %d floats the row buffers hold", width,
              200 * 1024 / 8);
  int threads = 32;
  while (threads < 512 && threads * 4 < width) threads <<= 1;
#define LAUNCH(T)                                                                                                  \
  do {                                                                                                             \
    if (smem > 48 * 1024)                                                                                          \
      NHV_CUDA(cudaFuncSetAttribute(postnorm_stream_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,        \
                                    (int)smem), "postnorm_stream");                                                \
    nhv_launch(postnorm_stream_kernel<T>, n_rows, threads, smem, stream, stream_rows, (T*)rounded, (const T*)a,    \
               (const T*)wa, ca, (const T*)b, (const T*)wb, cb, (const T*)w, (const T*)ls, width, eps, side_eps);  \
  } while (0)
  if (dtype == NHV_F32) LAUNCH(float);
  else if (dtype == NHV_BF16) LAUNCH(__nv_bfloat16);
  else NHV_REQUIRE(false, "postnorm_stream: unknown dtype %d", dtype);
#undef LAUNCH
  NHV_CHECK_LAUNCH("postnorm_stream");
  return 0;
}

template <typename T>
__global__ void stream_round_kernel(T* __restrict__ out, const float* __restrict__ stream, size_t total) {
  pdl_prologue();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_f32<T>(stream[i]);
}

NHV_API int nhv_stream_round(int dtype, void* out, const float* stream_rows, size_t total, cudaStream_t stream) {
  if (total == 0) return 0;
  const int threads = 256;
  const size_t want = (total + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  if (dtype == NHV_F32) nhv_launch(stream_round_kernel<float>, blocks, threads, 0, stream, (float*)out, stream_rows, total);
  else if (dtype == NHV_BF16)
    nhv_launch(stream_round_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (__nv_bfloat16*)out, stream_rows, total);
  else NHV_REQUIRE(false, "stream_round: unknown dtype %d", dtype);
  NHV_CHECK_LAUNCH("stream_round");
  return 0;
}
