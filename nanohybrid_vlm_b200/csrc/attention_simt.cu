// Causal grouped-query attention over cache pages, for any step shape: one kernel serves
// prompt portions and single decoded tokens alike, in fp32 or bf16 storage with all
// arithmetic in fp32.  It is the exact path (true 32-bit) and the fallback of the bf16
// path for head sizes and page sizes that the tensor-core kernels refuse.
//
// Replaces the two library calls at nanovllm/layers/attention.py:67-74.  Scores are
// (q . k) * scale, softmax over keys 0..pos of the same request (or the last `window`
// of them), query head h reads KV head h / (nq / nkv).
//
// The arithmetic for one (query token, head) is fixed: keys are visited in chunks of 32
// aligned to absolute multiples of 32, each dot product runs over the head size in
// ascending order, and the running maximum / sum / output are rescaled once per chunk.
// So a position's result does not depend on how tokens were cut into steps, on the
// batch around it, or on which pages hold the keys.
//
// Block = (tile of TQ consecutive new tokens of one request) x (one KV head) x (a
// sub-group of GS query heads that share it).  A "pair" is (token of the tile, head of
// the sub-group); pairs are dealt to the 4 warps round-robin, lane <-> key inside a
// chunk for the scores, lane <-> output column for the weighted sum of values.
//
// Two generalisations (nhv_attention_simt_ex): value heads of another size than key heads (dv; a page row holds
// `row` >= max(d, dv) elements and each kind uses its leading ones), and a sink per query head: a number that joins
// the softmax denominator as exp(sink) with no key, no value and no scale, counted once.  It enters as the start
// of the running maximum and sum (m = sink, l = 1), which later chunks rescale like any other term.
// Two more: a bias by distance, score - slopes[head] * (query position - key position), and pages with one plane
// (planes == 1): a row of such a page is the key, and its leading dv elements are the value as well (keys and
// values that are one latent vector per token, stored once).
// And kept first keys (keep_first, with a window): a query also sees the keys at positions below keep_first, at their
// true positions; their chunks are visited before the window's.
#include <math.h>

#include "nhv_common.cuh"

constexpr int AT_WARPS = 4;
constexpr int AT_CHUNK = 32;
constexpr int AT_MAX_D = 2048;
constexpr int AT_ACC = 64;              // output accumulators per lane: (pairs per warp) x (columns per lane)

// COLS: output columns per lane (value heads of up to 32 COLS elements); a warp then carries AT_ACC / COLS pairs.
template <typename T, int COLS>
__global__ void attn_paged_simt_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                                       const T* __restrict__ kv_pages, const int* __restrict__ block_table,
                                       int bt_stride, const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                                       int n_seqs, int nq, int nkv, int d, int page_size, int n_pages, int window,
                                       float scale, int TQ, int GS, int dv, int row, const float* __restrict__ sinks,
                                       int chunk, const float* __restrict__ slopes, int planes, int keep_first) {
  extern __shared__ float smem[];
  constexpr int AT_COLS = COLS, AT_PAIRS_PER_WARP = AT_ACC / COLS, AT_MAX_PAIRS = AT_PAIRS_PER_WARP * AT_WARPS;
  pdl_prologue();
  const int G = nq / nkv;
  const int kvh = blockIdx.y;
  const int g0 = blockIdx.z * GS;
  const int gs = min(GS, G - g0);

  // Which request and which tile of its new tokens is this block?
  int seq = -1, tile = blockIdx.x;
  for (int s = 0; s < n_seqs; ++s) {
    const int n = cu_q[s + 1] - cu_q[s];
    const int nt = (n + TQ - 1) / TQ;
    if (tile < nt) { seq = s; break; }
    tile -= nt;
  }
  if (seq < 0) return;
  const int n_new = cu_q[seq + 1] - cu_q[seq];
  const int total = kv_len[seq];
  const int q_pos0 = total - n_new;           // position of the request's first new token
  const int t0 = tile * TQ;                   // first token of the tile, within the new tokens
  const int tq_n = min(TQ, n_new - t0);
  const int n_pairs = tq_n * gs;
  const int pos_lo = q_pos0 + t0, pos_hi = q_pos0 + t0 + tq_n - 1;

  const int ks = d + 1;                        // padded key row: lane <-> key reads hit 32 banks
  float* Ks = smem;                            // [32][d+1]
  // one plane: the values are the keys' leading elements, read where the keys lie
  float* Vs = planes == 2 ? Ks + AT_CHUNK * ks : Ks;            // [32][dv]
  const int vs = planes == 2 ? dv : ks;
  float* Qs = Ks + AT_CHUNK * ks + (planes == 2 ? AT_CHUNK * dv : 0);      // [pairs][d]
  float* Ps = Qs + AT_MAX_PAIRS * d;           // [warps][32]
  __shared__ int key_ok[AT_CHUNK];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  for (int i = threadIdx.x; i < n_pairs * d; i += blockDim.x) {
    const int p = i / d, c = i - p * d;
    const int tq = p / gs, g = p - tq * gs;
    const size_t tok = (size_t)cu_q[seq] + t0 + tq;
    Qs[p * d + c] = to_f32<T>(q[tok * q_stride + (size_t)(kvh * G + g0 + g) * d + c]);
  }

  float m[AT_PAIRS_PER_WARP], l[AT_PAIRS_PER_WARP], o[AT_PAIRS_PER_WARP][AT_COLS];
#pragma unroll
  for (int i = 0; i < AT_PAIRS_PER_WARP; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
    const int p = warp + i * AT_WARPS;
    if (sinks && p < n_pairs) {
      m[i] = sinks[kvh * G + g0 + (p % gs)];
      l[i] = 1.f;
    }
#pragma unroll
    for (int c = 0; c < AT_COLS; ++c) o[i][c] = 0.f;
  }

  int first_key = 0;
  first_key = nhv_first_key(pos_lo, window, chunk);
  const int c_begin = (first_key / AT_CHUNK) * AT_CHUNK;
  // kept first keys: the chunks that hold keys [0, keep_first) come before the window's own chunks
  const int kept_end = keep_first > 0 ? min(((keep_first + AT_CHUNK - 1) / AT_CHUNK) * AT_CHUNK, c_begin) : 0;

  for (int c0 = kept_end > 0 ? 0 : c_begin; c0 <= pos_hi; c0 += AT_CHUNK) {
    if (c0 >= kept_end && c0 < c_begin) c0 = c_begin;
    __syncthreads();
    // Stage 32 keys and values (zero where there is no key or its page was given back).
    if (threadIdx.x < AT_CHUNK) {
      const int j = c0 + threadIdx.x;
      int ok = 0;
      if (j <= pos_hi && j < total) {
        const int page = block_table[(size_t)seq * bt_stride + j / page_size];
        ok = page >= 0 && page < n_pages;
      }
      key_ok[threadIdx.x] = ok;
    }
    __syncthreads();
    const int dmax = d > dv ? d : dv;
    for (int i = threadIdx.x; i < AT_CHUNK * dmax; i += blockDim.x) {
      const int r = i / dmax, c = i - r * dmax;
      float kx = 0.f, vx = 0.f;
      if (key_ok[r]) {
        const int j = c0 + r;
        const int page = block_table[(size_t)seq * bt_stride + j / page_size];
        const int off = j % page_size;
        const size_t base = ((((size_t)page * planes) * nkv + kvh) * page_size + off) * row + c;
        if (c < d) kx = to_f32<T>(kv_pages[base]);
        if (c < dv) vx = planes == 2 ? to_f32<T>(kv_pages[base + (size_t)nkv * page_size * row]) : (c < d ? kx : 0.f);
      }
      if (c < d) Ks[r * ks + c] = kx;
      if (planes == 2 && c < dv) Vs[r * dv + c] = vx;
    }
    __syncthreads();

#pragma unroll
    for (int i = 0; i < AT_PAIRS_PER_WARP; ++i) {
      const int p = warp + i * AT_WARPS;
      if (p >= n_pairs) break;
      const int tq = p / gs;
      const int pos = pos_lo + tq;
      const int lo = nhv_first_key(pos, window, chunk);
      if (c0 > pos || (c0 + AT_CHUNK <= lo && c0 >= keep_first)) continue;  // no key of this chunk is visible to this query
      const int j = c0 + lane;
      float s = -INFINITY;
      if (j <= pos && (j >= lo || j < keep_first) && key_ok[lane]) {
        const float* qv = Qs + p * d;
        const float* kv = Ks + lane * ks;
        float acc = 0.f;
        for (int c = 0; c < d; ++c) acc = fmaf(qv[c], kv[c], acc);
        s = acc * scale;
        if (slopes) s -= slopes[kvh * G + g0 + (p - tq * gs)] * (float)(pos - j);
      }
      const float cmax = warp_max(s);
      if (cmax == -INFINITY) continue;
      const float m_new = fmaxf(m[i], cmax);
      const float alpha = expf(m[i] - m_new);     // exp(-inf) = 0 on the first chunk
      const float pr = expf(s - m_new);           // 0 for masked keys
      l[i] = l[i] * alpha + warp_sum(pr);
      m[i] = m_new;
      Ps[warp * AT_CHUNK + lane] = pr;
      __syncwarp();
#pragma unroll
      for (int cc = 0; cc < AT_COLS; ++cc) {
        const int c = lane + cc * 32;
        if (c < dv) {
          float acc = 0.f;
          for (int r = 0; r < AT_CHUNK; ++r) acc = fmaf(Ps[warp * AT_CHUNK + r], Vs[r * vs + c], acc);
          o[i][cc] = o[i][cc] * alpha + acc;
        }
      }
      __syncwarp();
    }
  }

#pragma unroll
  for (int i = 0; i < AT_PAIRS_PER_WARP; ++i) {
    const int p = warp + i * AT_WARPS;
    if (p >= n_pairs) break;
    const int tq = p / gs, g = p - tq * gs;
    const size_t tok = (size_t)cu_q[seq] + t0 + tq;
    T* dst = out + tok * out_stride + (size_t)(kvh * G + g0 + g) * dv;
    const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
#pragma unroll
    for (int cc = 0; cc < AT_COLS; ++cc) {
      const int c = lane + cc * 32;
      if (c < dv) dst[c] = from_f32<T>(o[i][cc] * inv);
    }
  }
}

// max_tiles: an upper bound on sum over requests of ceil(new tokens / TQ); the caller may pass
// n_tokens / TQ + n_seqs.  Blocks beyond the true count leave at once.
NHV_API int nhv_attention_simt_ex(int dtype, const void* q, int q_stride, void* out, int out_stride,
                                  const void* kv_pages, const int* block_table, int bt_stride, const int* cu_q,
                                  const int* kv_len, int n_seqs, int n_tokens, int nq, int nkv, int d, int dv, int row,
                                  int page_size, int n_pages, int window, int chunk, float scale, const float* sinks,
                                  const float* slopes, int planes, int keep_first, cudaStream_t stream) {
  if (n_tokens == 0 || n_seqs == 0) return 0;
  NHV_REQUIRE(keep_first >= 0 && (keep_first == 0 || window > 0), "attention: kept first keys go with a window");
  NHV_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention: %d query heads do not divide into %d KV heads", nq, nkv);
  NHV_REQUIRE(d > 0 && d <= AT_MAX_D && dv > 0 && dv <= AT_MAX_D, "attention: head sizes %d / %d are beyond the supported %d",
              d, dv, AT_MAX_D);
  NHV_REQUIRE(row >= d && row >= dv, "attention: a page row of %d elements does not hold a head of %d / %d", row, d, dv);
  NHV_REQUIRE(page_size > 0 && n_pages > 0 && bt_stride > 0, "attention: bad page geometry");
  NHV_REQUIRE(planes == 2 || (planes == 1 && dv <= d), "attention: pages have a key and a value plane, or one plane whose rows' leading elements are the values");
  const int G = nq / nkv;
  const int cols = dv <= 256 ? 8 : dv <= 512 ? 16 : dv <= 1024 ? 32 : 64;
  const int max_pairs = AT_ACC / cols * AT_WARPS;
  const int GS = G < 8 ? (G < max_pairs ? G : max_pairs) : (8 < max_pairs ? 8 : max_pairs);
  const int TQ = max_pairs / GS;
  const int max_tiles = n_tokens / TQ + n_seqs;
  const size_t smem = ((size_t)AT_CHUNK * (d + 1) + (planes == 2 ? (size_t)AT_CHUNK * dv : 0) + (size_t)max_pairs * d +
                       AT_WARPS * AT_CHUNK) * sizeof(float);
  NHV_REQUIRE(smem <= 227 * 1024, "attention: head sizes %d / %d need %zu bytes of shared memory", d, dv, smem);
  dim3 grid(max_tiles, nkv, (G + GS - 1) / GS);
#define LAUNCH(T, COLS)                                                                                              \
  do {                                                                                                               \
    if (smem > 48 * 1024)                                                                                            \
      NHV_CUDA(cudaFuncSetAttribute(attn_paged_simt_kernel<T, COLS>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                    (int)smem), "attention");                                                        \
    nhv_launch(attn_paged_simt_kernel<T, COLS>, grid, AT_WARPS * 32, smem, stream,                                   \
        (const T*)q, q_stride, (T*)out, out_stride, (const T*)kv_pages, block_table, bt_stride, cu_q, kv_len,        \
        n_seqs, nq, nkv, d, page_size, n_pages, window, scale, TQ, GS, dv, row, sinks, chunk, slopes, planes,        \
        keep_first);                                                                                                 \
  } while (0)
#define LAUNCH_COLS(T)                 \
  do {                                 \
    if (cols == 8) LAUNCH(T, 8);       \
    else if (cols == 16) LAUNCH(T, 16); \
    else if (cols == 32) LAUNCH(T, 32); \
    else LAUNCH(T, 64);                \
  } while (0)
  if (dtype == NHV_F32) LAUNCH_COLS(float);
  else if (dtype == NHV_BF16) LAUNCH_COLS(__nv_bfloat16);
  else NHV_REQUIRE(false, "attention: unknown dtype %d", dtype);
#undef LAUNCH_COLS
#undef LAUNCH
  NHV_CHECK_LAUNCH("attention");
  return 0;
}

NHV_API int nhv_attention_simt(int dtype, const void* q, int q_stride, void* out, int out_stride,
                               const void* kv_pages, const int* block_table, int bt_stride, const int* cu_q,
                               const int* kv_len, int n_seqs, int n_tokens, int nq, int nkv, int d, int page_size,
                               int n_pages, int window, float scale, cudaStream_t stream) {
  return nhv_attention_simt_ex(dtype, q, q_stride, out, out_stride, kv_pages, block_table, bt_stride, cu_q, kv_len,
                               n_seqs, n_tokens, nq, nkv, d, d, d, page_size, n_pages, window, 0, scale, nullptr, nullptr, 2, 0, stream);
}
