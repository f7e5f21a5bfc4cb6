// A residual stream kept in 32-bit floats while the layers compute in the storage type.
//
//   embed_scaled_f32:  stream[t] = table[ids[t]] * scale                       (fp32 out)
//   rmsnorm_stream:    s = stream[src] + c0 a0[src] + c1 a1[src] + c2 a2[src]  (addends optional; all sums in fp32)
//                      stream[src] = s                                         (if write_stream)
//                      out[r] = s / sqrt(mean(s^2) + eps) * (w + weight_offset), rounded once to the storage type
//                      src = rows[r] or r
//                      groups > 1: the row is cut into that many equal consecutive parts and each part is divided
//                      by the root mean square of its own elements
// One block per row; the row of fp32 sums lives in shared memory between the two passes.
#include "nhv_common.cuh"

template <typename T>
__global__ void embed_scaled_f32_kernel(float* __restrict__ out, const T* __restrict__ table,
                                        const int* __restrict__ ids, int width, int vocab, float scale) {
  pdl_prologue();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  const T* src = table + (size_t)(ok ? id : 0) * width;
  float* dst = out + (size_t)t * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = ok ? to_f32<T>(src[c]) * scale : 0.f;
}

NHV_API int nhv_embed_scaled_f32(int dtype, float* out, const void* table, const int* ids, int n_tokens, int width,
                                 int vocab, float scale, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  NHV_REQUIRE(n_tokens > 0 && width > 0 && vocab > 0, "embed_scaled_f32: bad sizes");
  const int threads = width >= 1024 ? 256 : 128;
  if (dtype == NHV_F32)
    nhv_launch(embed_scaled_f32_kernel<float>, n_tokens, threads, 0, stream, out, (const float*)table, ids, width, vocab, scale);
  else if (dtype == NHV_BF16)
    nhv_launch(embed_scaled_f32_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, out, (const __nv_bfloat16*)table, ids,
               width, vocab, scale);
  else
    NHV_REQUIRE(false, "embed_scaled_f32: unknown dtype %d", dtype);
  NHV_CHECK_LAUNCH("embed_scaled_f32");
  return 0;
}

template <typename T>
__global__ void rmsnorm_stream_kernel(T* __restrict__ out, const T* __restrict__ a0, const T* __restrict__ a1,
                                      const T* __restrict__ a2, float c0, float c1, float c2,
                                      float* __restrict__ stream, const T* __restrict__ w,
                                      const int* __restrict__ rows, int width, float eps, int write_stream,
                                      float weight_offset, int groups) {
  extern __shared__ float row[];
  __shared__ float red[33];
  pdl_prologue();
  const int r = blockIdx.x;
  const size_t src = (size_t)(rows ? rows[r] : r) * width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float s = stream[src + c];
    if (a0) {
      float add = c0 * to_f32<T>(a0[src + c]);
      if (a1) add = fmaf(c1, to_f32<T>(a1[src + c]), add);
      if (a2) add = fmaf(c2, to_f32<T>(a2[src + c]), add);
      s += add;
      if (write_stream) stream[src + c] = s;
    }
    row[c] = s;
    ss = fmaf(s, s, ss);
  }
  T* dst = out + (size_t)r * width;
  if (groups > 1) {
    // one warp per part in turn: the part's sum of squares in a fixed order, then its outputs
    __syncthreads();
    const int part = width / groups, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    for (int g = warp; g < groups; g += nwarp) {
      const float* pr = row + (size_t)g * part;
      float sg = 0.f;
      for (int c = lane; c < part; c += 32) sg = fmaf(pr[c], pr[c], sg);
      sg = warp_sum(sg);
      const float rg = 1.0f / sqrtf(sg / (float)part + eps);
      for (int c = lane; c < part; c += 32)
        dst[g * part + c] = from_f32<T>(pr[c] * rg * (to_f32<T>(w[g * part + c]) + weight_offset));
    }
    return;
  }
  const float total = block_sum(ss, red);
  const float rstd = 1.0f / sqrtf(total / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    dst[c] = from_f32<T>(row[c] * rstd * (to_f32<T>(w[c]) + weight_offset));
}

NHV_API int nhv_rmsnorm_stream(int dtype, void* out, const void* a0, const void* a1, const void* a2, float c0, float c1,
                               float c2, float* stream_rows, const void* w, const int* rows, int n_rows, int width,
                               float eps, int write_stream, float weight_offset, int groups, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NHV_REQUIRE(n_rows > 0 && width > 0 && stream_rows && out && w, "rmsnorm_stream: bad arguments");
  NHV_REQUIRE(groups >= 1 && width % groups == 0, "rmsnorm_stream: a row of %d does not divide into %d parts", width, groups);
  NHV_REQUIRE((a0 || !a1) && (a1 || !a2), "rmsnorm_stream: addends are given in order");
  NHV_REQUIRE(!(rows && write_stream), "rmsnorm_stream: a gathered norm cannot write the stream back");
  const size_t smem = (size_t)width * sizeof(float);
  NHV_REQUIRE(smem <= 200 * 1024, "rmsnorm_stream: width %d is beyond the %d floats a row buffer holds", width, 200 * 1024 / 4);
  int threads = 32;
  while (threads < 512 && threads * 4 < width) threads <<= 1;
#define LAUNCH(T)                                                                                               \
  do {                                                                                                          \
    if (smem > 48 * 1024)                                                                                       \
      NHV_CUDA(cudaFuncSetAttribute(rmsnorm_stream_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                                    (int)smem), "rmsnorm_stream");                                              \
    nhv_launch(rmsnorm_stream_kernel<T>, n_rows, threads, smem, stream, (T*)out, (const T*)a0, (const T*)a1,    \
               (const T*)a2, c0, c1, c2, stream_rows, (const T*)w, rows, width, eps, write_stream, weight_offset, groups); \
  } while (0)
  if (dtype == NHV_F32) LAUNCH(float);
  else if (dtype == NHV_BF16) LAUNCH(__nv_bfloat16);
  else NHV_REQUIRE(false, "rmsnorm_stream: unknown dtype %d", dtype);
#undef LAUNCH
  NHV_CHECK_LAUNCH("rmsnorm_stream");
  return 0;
}

// out = ca * a + cb * b, elementwise, sums in fp32.
template <typename T>
__global__ void scaled_sum_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b, float ca,
                                  float cb, size_t total) {
  pdl_prologue();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_f32<T>(fmaf(cb, to_f32<T>(b[i]), ca * to_f32<T>(a[i])));
}

NHV_API int nhv_scaled_sum(int dtype, void* out, const void* a, const void* b, float ca, float cb, size_t total,
                           cudaStream_t stream) {
  if (total == 0) return 0;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  if (dtype == NHV_F32)
    nhv_launch(scaled_sum_kernel<float>, blocks, threads, 0, stream, (float*)out, (const float*)a, (const float*)b, ca, cb, total);
  else if (dtype == NHV_BF16)
    nhv_launch(scaled_sum_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)a,
               (const __nv_bfloat16*)b, ca, cb, total);
  else
    NHV_REQUIRE(false, "scaled_sum: unknown dtype %d", dtype);
  NHV_CHECK_LAUNCH("scaled_sum");
  return 0;
}
