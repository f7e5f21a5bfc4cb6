// Rotary position encoding, then a unit-RMS norm without a weight, then the key/value store, for attention whose
// key and value heads may differ in size.
//
// One warp per (token, head) of the packed projection output qkv [T, nq*dk + nkv*dk + nkv*dv]:
//   q heads: rotate the first rotary_dim elements (element i with i + rotary_dim/2, angle from the table), then
//            x / sqrt(mean(x^2) + eps) over the head -> q_out [T, nq, dk]
//   k heads: the same -> the token's slot of the K pages
//   v heads: copied -> the token's slot of the V pages
// eps < 0 leaves the norm out.  Rotation and norm are computed in fp32 and rounded once.
// norm_first: the norm (with its weight) comes before the rotation instead of after it.  interleaved: element 2i turns
// with element 2i + 1 (the table is the same: cos then sin of angle i).
// q_weight / k_weight (optional, [dk], shared by the heads of their kind): the normed head times this weight.
// bias (optional, [nq*dk + nkv*dk], the query and key columns of qkv): added in fp32 to what the projection gave,
// before anything else (projected values have none).  v_from_k: the values are the key heads as projected (with their bias, before the rotation); qkv
// then has no value columns and dv == dk.
// Cache pages of one layer: [page][K|V][kv_head][slot_in_page][row], row >= max(dk, dv); the elements of a row
// beyond the head's size are cleared.  slot_mapping[t] = page * page_size + slot_in_page, or -1 for "do not store".
#include "nhv_common.cuh"

constexpr int RN_WARPS = 4;
constexpr int RN_MAX_D = 512;

template <typename T>
__global__ void rope_norm_store_kernel(const T* __restrict__ qkv, int qkv_stride, T* __restrict__ q_out,
                                       int q_out_stride, T* __restrict__ kv_pages,
                                       const int* __restrict__ slot_mapping, const int* __restrict__ positions,
                                       const float* __restrict__ cos_sin, int rotary_dim, int max_position,
                                       int n_tokens, int nq, int nkv, int dk, int dv, int row, int page_size,
                                       int n_pages, float eps, int heads_per_token, const T* __restrict__ bias,
                                       int v_from_k, const T* __restrict__ q_weight,
                                       const T* __restrict__ k_weight, int norm_first, int interleaved) {
  extern __shared__ float smem[];
  pdl_prologue();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * RN_WARPS + warp;
  if (item >= (long)n_tokens * heads_per_token) return;
  const int t = (int)(item / heads_per_token);
  const int head = (int)(item - (long)t * heads_per_token);
  float* v = smem + warp * RN_MAX_D;
  const int kind = head < nq ? 0 : (head < nq + nkv ? 1 : 2);  // q, k, v
  const int d = kind == 2 ? dv : dk;
  const size_t col0 = kind == 2 ? (v_from_k ? (size_t)(head - nkv) * dk : (size_t)(nq + nkv) * dk + (size_t)(head - nq - nkv) * dv)
                                : (size_t)head * dk;
  const T* src = qkv + (size_t)t * qkv_stride + col0;
  T* dst;
  int width = d;
  if (kind == 0) {
    dst = q_out + (size_t)t * q_out_stride + (size_t)head * dk;
  } else {
    const int slot = slot_mapping[t];
    if (slot < 0 || slot >= n_pages * page_size) return;
    const int page = slot / page_size, off = slot - page * page_size;
    const int kvh = kind == 1 ? head - nq : head - nq - nkv;
    dst = kv_pages + ((((size_t)page * 2 + (kind - 1)) * nkv + kvh) * page_size + off) * row;
    width = row;
  }
  if (bias && (kind != 2 || v_from_k)) {
    for (int c = lane; c < d; c += 32) v[c] = to_f32<T>(src[c]) + to_f32<T>(bias[col0 + c]);
  } else {
    for (int c = lane; c < d; c += 32) v[c] = to_f32<T>(src[c]);
  }
  __syncwarp();
  float ss = 0.f;
  float mine[RN_MAX_D / 32];
  if (kind != 2) {
    const T* hw = kind == 0 ? q_weight : k_weight;
    if (norm_first && eps >= 0.f) {
      // the norm (and its weight) before the rotation: the head in shared memory is replaced by its normed self
      float s0 = 0.f;
      for (int c = lane; c < d; c += 32) s0 = fmaf(v[c], v[c], s0);
      s0 = warp_sum(s0);
      const float r0 = 1.0f / sqrtf(s0 / (float)d + eps);
      for (int c = lane; c < d; c += 32) v[c] = hw ? v[c] * r0 * to_f32<T>(hw[c]) : v[c] * r0;
      __syncwarp();
    }
    const float* cs = nullptr;
    const int half = rotary_dim >> 1;
    if (cos_sin) {
      int pos = positions[t];
      pos = pos < 0 ? 0 : (pos >= max_position ? max_position - 1 : pos);
      cs = cos_sin + (size_t)pos * rotary_dim;                  // cos[0..half) then sin[0..half)
    }
#pragma unroll
    for (int k = 0; k < RN_MAX_D / 32; ++k) {
      const int c = lane + k * 32;
      float yv = 0.f;
      if (c < d) {
        yv = v[c];
        if (cs && interleaved && c < rotary_dim) {
          const int i = c >> 1;                                 // the pair (2i, 2i + 1) turns by angle i
          yv = (c & 1) ? v[c] * cs[i] + v[c - 1] * cs[half + i] : v[c] * cs[i] - v[c + 1] * cs[half + i];
        } else if (cs && c < half) yv = v[c] * cs[c] - v[c + half] * cs[half + c];
        else if (cs && c < rotary_dim) yv = v[c] * cs[c - half] + v[c - half] * cs[c];
        ss = fmaf(yv, yv, ss);
      }
      mine[k] = yv;
    }
    ss = warp_sum(ss);
    const float r = eps >= 0.f && !norm_first ? 1.0f / sqrtf(ss / (float)d + eps) : 1.0f;
    if (norm_first) hw = nullptr;
#pragma unroll
    for (int k = 0; k < RN_MAX_D / 32; ++k) {
      const int c = lane + k * 32;
      if (c < d) dst[c] = from_f32<T>(hw ? mine[k] * r * to_f32<T>(hw[c]) : mine[k] * r);
    }
  } else {
    for (int c = lane; c < d; c += 32) dst[c] = from_f32<T>(v[c]);
  }
  for (int c = d + lane; c < width; c += 32) dst[c] = from_f32<T>(0.f);
}

NHV_API int nhv_rope_norm_store(int dtype, const void* qkv, int qkv_stride, void* q_out, int q_out_stride,
                                void* kv_pages, const int* slot_mapping, const int* positions, const float* cos_sin,
                                int rotary_dim, int max_position, int n_tokens, int nq, int nkv, int dk, int dv, int row,
                                int page_size, int n_pages, float eps, const void* bias, int v_from_k,
                                const void* q_weight, const void* k_weight, int norm_first, int interleaved,
                                cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  NHV_REQUIRE(n_tokens > 0 && nq > 0 && nkv >= 0 && dk > 0 && dv > 0, "rope_norm_store: bad sizes");
  NHV_REQUIRE(dk <= RN_MAX_D && dv <= RN_MAX_D, "rope_norm_store: head sizes %d / %d are beyond the supported %d", dk, dv, RN_MAX_D);
  NHV_REQUIRE(!cos_sin || (rotary_dim > 0 && rotary_dim % 2 == 0 && rotary_dim <= dk),
              "rope_norm_store: rotary_dim %d must be even and at most the head size %d", rotary_dim, dk);
  NHV_REQUIRE(kv_pages == nullptr || (page_size > 0 && n_pages > 0 && slot_mapping && row >= dk && row >= dv),
              "rope_norm_store: a key/value store needs pages whose rows hold a head, and a slot mapping");
  NHV_REQUIRE(!cos_sin || positions, "rope_norm_store: rotation needs positions");
  NHV_REQUIRE(!v_from_k || dv == dk, "rope_norm_store: values taken from the keys have the keys' size, not %d", dv);
  const int heads_per_token = kv_pages ? nq + 2 * nkv : nq;
  const long items = (long)n_tokens * heads_per_token;
  const int blocks = (int)((items + RN_WARPS - 1) / RN_WARPS);
  const size_t smem = (size_t)RN_WARPS * RN_MAX_D * sizeof(float);
#define LAUNCH(T)                                                                                                  \
  nhv_launch(rope_norm_store_kernel<T>, blocks, RN_WARPS * 32, smem, stream, (const T*)qkv, qkv_stride, (T*)q_out, \
             q_out_stride, (T*)kv_pages, slot_mapping, positions, cos_sin, rotary_dim, max_position, n_tokens, nq, \
             nkv, dk, dv, row, page_size, n_pages, eps, heads_per_token, (const T*)bias, v_from_k, (const T*)q_weight,    \
             (const T*)k_weight, norm_first, interleaved)
  if (dtype == NHV_F32) LAUNCH(float);
  else if (dtype == NHV_BF16) LAUNCH(__nv_bfloat16);
  else NHV_REQUIRE(false, "rope_norm_store: unknown dtype %d", dtype);
#undef LAUNCH
  NHV_CHECK_LAUNCH("rope_norm_store");
  return 0;
}
