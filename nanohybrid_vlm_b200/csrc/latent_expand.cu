// Attention over one latent per token, prompt portions in bfloat16: the latents of a step's requests are expanded
// into keys and values per head once, so that the tensor-core attention kernels can run over them (for a portion of
// many tokens that costs far fewer operations than attending over the latents themselves, whose rows are several
// times a head's size).
//
// Temporary rows: request s owns rows [row0[s], row0[s] + 64 * ceil(kv_len[s] / 64)), row0 a multiple of 64, so that
// 64 rows are one temporary page.
//
// latent_gather:    cache pages with one plane ([page][1][1][slot][row]: latent [rank], rotated key part [dr]) ->
//                   lat [rows, rank] and kr [rows, dr], contiguous; rows past a request's last token are cleared, so
//                   that the product that follows makes zeros, not whatever the memory held.
// (a library product expands lat with the stacked matrices [H dn + H dv, rank] into kv [rows, H dn + H dv])
// latent_assemble:  kv and kr -> temporary pages [page][2][H][64][D]: the key of head h is [kv's H dn part | kr | 0],
//                   its value [kv's H dv part | 0]; and the step's queries q [T, H, dn + dr] (unrotated part) with
//                   q_lat [T, H, rank + dr] (whose last dr elements are the rotated part) -> qp [T, H, D], zero padded.
#include "nhv_common.cuh"

constexpr int LE_TILE = 64;     // rows of a temporary page

template <typename T>
__global__ void latent_gather_kernel(T* __restrict__ lat, T* __restrict__ kr, const T* __restrict__ pages,
                                     const int* __restrict__ block_table, int bt_stride, const int* __restrict__ kv_len,
                                     const int* __restrict__ row0, int rank, int dr, int row, int page_size, int n_pages) {
  pdl_prologue();
  const int s = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total = kv_len[s];
  const int padded = (total + LE_TILE - 1) / LE_TILE * LE_TILE;
  const int j = blockIdx.x * (blockDim.x >> 5) + warp;
  if (j >= padded) return;
  const size_t r = (size_t)row0[s] + j;
  const T* src = nullptr;
  if (j < total) {
    const int page = block_table[(size_t)s * bt_stride + j / page_size];
    if (page >= 0 && page < n_pages) src = pages + ((size_t)page * page_size + j % page_size) * row;
  }
  for (int c = lane; c < rank; c += 32) lat[r * rank + c] = src ? src[c] : from_f32<T>(0.f);
  for (int c = lane; c < dr; c += 32) kr[r * dr + c] = src ? src[rank + c] : from_f32<T>(0.f);
}

template <typename T>
__global__ void latent_assemble_kernel(T* __restrict__ tmp, T* __restrict__ qp, const T* __restrict__ kv,
                                       const T* __restrict__ kr, const T* __restrict__ q, int q_stride,
                                       const T* __restrict__ q_lat, int q_lat_stride, size_t n_rows, int n_tokens, int H,
                                       int dn, int dr, int dv, int rank, int D) {
  pdl_prologue();
  const size_t per_row = (size_t)H * D;
  const size_t n_kv = n_rows * per_row, total = 2 * n_kv + (size_t)n_tokens * per_row;
  const int kvw = H * (dn + dv);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    if (i < 2 * n_kv) {
      const int plane = i >= n_kv;
      const size_t e = i - (plane ? n_kv : 0);
      const size_t r = e / per_row;
      const int h = (int)((e - r * per_row) / D), c = (int)(e - r * per_row - (size_t)h * D);
      T v = from_f32<T>(0.f);
      if (plane == 0) {
        if (c < dn) v = kv[r * kvw + (size_t)h * dn + c];
        else if (c < dn + dr) v = kr[r * dr + (c - dn)];
      } else if (c < dv) {
        v = kv[r * kvw + (size_t)H * dn + (size_t)h * dv + c];
      }
      const size_t page = r / LE_TILE, slot = r - page * LE_TILE;
      tmp[(((page * 2 + plane) * H + h) * LE_TILE + slot) * D + c] = v;
    } else {
      const size_t e = i - 2 * n_kv;
      const size_t t = e / per_row;
      const int h = (int)((e - t * per_row) / D), c = (int)(e - t * per_row - (size_t)h * D);
      T v = from_f32<T>(0.f);
      if (c < dn) v = q[t * q_stride + (size_t)h * (dn + dr) + c];
      else if (c < dn + dr) v = q_lat[t * q_lat_stride + (size_t)h * (rank + dr) + rank + (c - dn)];
      qp[e] = v;
    }
  }
}

NHV_API int nhv_latent_gather(int dtype, void* lat, void* kr, const void* pages, const int* block_table, int bt_stride,
                              const int* kv_len, const int* row0, int n_seqs, int max_kv_len, int rank, int dr, int row,
                              int page_size, int n_pages, cudaStream_t stream) {
  if (n_seqs == 0 || max_kv_len == 0) return 0;
  NHV_REQUIRE(rank > 0 && dr >= 0 && row >= rank + dr && page_size > 0 && n_pages > 0 && bt_stride > 0,
              "latent_gather: bad sizes");
  const int warps = 8;
  const int padded = (max_kv_len + LE_TILE - 1) / LE_TILE * LE_TILE;
  dim3 grid((padded + warps - 1) / warps, n_seqs);
#define LAUNCH(T)                                                                                                       \
  nhv_launch(latent_gather_kernel<T>, grid, warps * 32, 0, stream, (T*)lat, (T*)kr, (const T*)pages, block_table,        \
             bt_stride, kv_len, row0, rank, dr, row, page_size, n_pages)
  if (dtype == NHV_F32) LAUNCH(float);
  else if (dtype == NHV_BF16) LAUNCH(__nv_bfloat16);
  else NHV_REQUIRE(false, "latent_gather: unknown dtype %d", dtype);
#undef LAUNCH
  NHV_CHECK_LAUNCH("latent_gather");
  return 0;
}

NHV_API int nhv_latent_assemble(int dtype, void* tmp, void* qp, const void* kv, const void* kr, const void* q, int q_stride,
                                const void* q_lat, int q_lat_stride, long n_rows, int n_tokens, int H, int dn, int dr,
                                int dv, int rank, int D, cudaStream_t stream) {
  if (n_rows == 0 && n_tokens == 0) return 0;
  NHV_REQUIRE(H > 0 && dn >= 0 && dr >= 0 && dv > 0 && D >= dn + dr && D >= dv && n_rows % LE_TILE == 0,
              "latent_assemble: a padded head of %d elements must hold the key's %d and the value's %d", D, dn + dr, dv);
  const size_t total = (2 * (size_t)n_rows + (size_t)n_tokens) * H * D;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
#define LAUNCH(T)                                                                                                    \
  nhv_launch(latent_assemble_kernel<T>, blocks, 256, 0, stream, (T*)tmp, (T*)qp, (const T*)kv, (const T*)kr,          \
             (const T*)q, q_stride, (const T*)q_lat, q_lat_stride, (size_t)n_rows, n_tokens, H, dn, dr, dv, rank, D)
  if (dtype == NHV_F32) LAUNCH(float);
  else if (dtype == NHV_BF16) LAUNCH(__nv_bfloat16);
  else NHV_REQUIRE(false, "latent_assemble: unknown dtype %d", dtype);
#undef LAUNCH
  NHV_CHECK_LAUNCH("latent_assemble");
  return 0;
}
