// Attention whose keys and values are one latent vector per token: what a token leaves in the cache, and the rotated
// part of its queries.
//
// One warp per (token, item).  Item 0 takes the token's row kv [rank + dr] of the down projection: the first `rank`
// elements are divided by their root mean square (eps inside the root) and multiplied by a weight [rank]: the latent;
// the last dr elements are one key part shared by all heads, of which the first rotary_dim rotate (element i with
// i + rotary_dim / 2, angles from the table).  Both go to the token's slot of a page with one plane,
// [page][1][1][slot_in_page][row], row >= rank + dr, latent first; the rest of the row is cleared.
// Items 1 .. H take head h of q [T, H, dn + dr]: its last dr elements, rotated the same way, go to
// q_lat [T, H, rank + dr] behind the `rank` elements that a product with the keys' expansion fills.
// Norm and rotation are computed in fp32 and rounded once.
#include "nhv_common.cuh"

constexpr int LS_WARPS = 4;
constexpr int LS_MAX_ROW = 2048;

template <typename T>
__global__ void latent_rope_store_kernel(const T* __restrict__ kv, int kv_stride, const T* __restrict__ q, int q_stride,
                                         T* __restrict__ q_lat, int q_lat_stride, T* __restrict__ pages,
                                         const int* __restrict__ slot_mapping, const int* __restrict__ positions,
                                         const float* __restrict__ cos_sin, int rotary_dim, int max_position,
                                         int n_tokens, int H, int dn, int dr, int rank, int row, int page_size,
                                         int n_pages, float eps, const T* __restrict__ weight) {
  extern __shared__ float smem[];
  pdl_prologue();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * LS_WARPS + warp;
  if (item >= (long)n_tokens * (H + 1)) return;
  const int t = (int)(item / (H + 1));
  const int which = (int)(item - (long)t * (H + 1));
  float* v = smem + (size_t)warp * (rank + dr);
  const float* cs = nullptr;
  const int half = rotary_dim >> 1;
  if (cos_sin) {
    int pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= max_position ? max_position - 1 : pos);
    cs = cos_sin + (size_t)pos * rotary_dim;                    // cos[0..half) then sin[0..half)
  }
  auto turned = [&](const float* x, int c) {                    // element c of the rotated part x [dr]
    if (cs && c < half) return x[c] * cs[c] - x[c + half] * cs[half + c];
    if (cs && c < rotary_dim) return x[c] * cs[c - half] + x[c - half] * cs[c];
    return x[c];
  };
  if (which == 0) {
    if (!pages) return;
    const int slot = slot_mapping[t];
    if (slot < 0 || slot >= n_pages * page_size) return;
    const T* src = kv + (size_t)t * kv_stride;
    for (int c = lane; c < rank + dr; c += 32) v[c] = to_f32<T>(src[c]);
    __syncwarp();
    float ss = 0.f;
    for (int c = lane; c < rank; c += 32) ss = fmaf(v[c], v[c], ss);
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)rank + eps);
    T* dst = pages + (size_t)slot * row;
    for (int c = lane; c < rank; c += 32) dst[c] = from_f32<T>(v[c] * r * to_f32<T>(weight[c]));
    for (int c = lane; c < dr; c += 32) dst[rank + c] = from_f32<T>(turned(v + rank, c));
    for (int c = rank + dr + lane; c < row; c += 32) dst[c] = from_f32<T>(0.f);
  } else {
    const int h = which - 1;
    const T* src = q + (size_t)t * q_stride + (size_t)h * (dn + dr) + dn;
    for (int c = lane; c < dr; c += 32) v[c] = to_f32<T>(src[c]);
    __syncwarp();
    T* dst = q_lat + (size_t)t * q_lat_stride + (size_t)h * (rank + dr) + rank;
    for (int c = lane; c < dr; c += 32) dst[c] = from_f32<T>(turned(v, c));
  }
}

NHV_API int nhv_latent_rope_store(int dtype, const void* kv, int kv_stride, const void* q, int q_stride, void* q_lat,
                                  int q_lat_stride, void* pages, const int* slot_mapping, const int* positions,
                                  const float* cos_sin, int rotary_dim, int max_position, int n_tokens, int H, int dn,
                                  int dr, int rank, int row, int page_size, int n_pages, float eps, const void* weight,
                                  cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  NHV_REQUIRE(n_tokens > 0 && H > 0 && dn >= 0 && dr >= 0 && rank > 0, "latent_rope_store: bad sizes");
  NHV_REQUIRE(rank + dr <= LS_MAX_ROW, "latent_rope_store: a row of %d elements is beyond the supported %d", rank + dr, LS_MAX_ROW);
  NHV_REQUIRE(!cos_sin || (rotary_dim > 0 && rotary_dim % 2 == 0 && rotary_dim <= dr && positions),
              "latent_rope_store: rotary_dim %d must be even and at most the rotated part %d, and needs positions", rotary_dim, dr);
  NHV_REQUIRE(pages == nullptr || (page_size > 0 && n_pages > 0 && slot_mapping && row >= rank + dr && weight),
              "latent_rope_store: the store needs pages whose rows hold the latent and the rotated part, a slot mapping and the norm's weight");
  const long items = (long)n_tokens * (H + 1);
  const int blocks = (int)((items + LS_WARPS - 1) / LS_WARPS);
  const size_t smem = (size_t)LS_WARPS * (rank + dr) * sizeof(float);
#define LAUNCH(T)                                                                                                   \
  nhv_launch(latent_rope_store_kernel<T>, blocks, LS_WARPS * 32, smem, stream, (const T*)kv, kv_stride, (const T*)q, \
             q_stride, (T*)q_lat, q_lat_stride, (T*)pages, slot_mapping, positions, cos_sin, rotary_dim,            \
             max_position, n_tokens, H, dn, dr, rank, row, page_size, n_pages, eps, (const T*)weight)
  if (dtype == NHV_F32) LAUNCH(float);
  else if (dtype == NHV_BF16) LAUNCH(__nv_bfloat16);
  else NHV_REQUIRE(false, "latent_rope_store: unknown dtype %d", dtype);
#undef LAUNCH
  NHV_CHECK_LAUNCH("latent_rope_store");
  return 0;
}
