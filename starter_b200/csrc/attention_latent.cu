// Attention over a cached low-rank latent (multi-head latent attention) with a sliding window.
//
// Per token the cache holds ONE row for all heads: the normed latent c (`rank` entries) followed by a
// rotated key part (`rot` entries) that every head shares.  A head's key is [W_uk c | shared part] and
// its value W_uv c.  Nothing of W_uk and W_uv is applied to the cache here: the caller folds W_uk into
// the query (q' = W_uk^T q_plain, `rank` entries) and applies W_uv to the output, so that
//
//     score(t, s) = (q'_t . c_s + q_rot_t . shared_s) * scale,     o'_t = sum_s softmax(score)_s c_s
//
// and the kernel sees queries of rank + rot entries, keys that are the cache rows and values that are
// their first `rank` entries.  A query at position p sees s with 0 <= p - s < window (window <= 0: all
// s <= p).
//
// latent_prepare: what follows the stacked down-projections of a token.  The query latent is
// RMS-normed (gain qg) into cq; the key/value latent is RMS-normed (gain kg) and filed in the cache
// row of the token's position; the shared key part is turned by the token's position and filed behind
// it.  latent_rotate_q turns the rotated part of every head's query and files it behind q'.
// Rotation: pairs (2i, 2i + 1) of the first rot_dims entries, by the angle whose cos and sin the
// tables hold at [position][i]; entries from rot_dims on pass unchanged.  Norms, angles, scores, the
// softmax and the sums over keys are float.
#include "common.cuh"

template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ proj, int proj_width, const float* __restrict__ qg,
                                      const float* __restrict__ kg, float eps, const float* __restrict__ cos_t,
                                      const float* __restrict__ sin_t, int table_width,
                                      const int* __restrict__ tok_pos, const int* __restrict__ tok_slot,
                                      const int* __restrict__ block_table, int table_stride, T* __restrict__ store,
                                      T* __restrict__ cq, int q_rank, int rank, int rot, int rot_dims, int write) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(proj);
  SB_BEHIND_WAIT(tok_pos);
  SB_BEHIND_WAIT(tok_slot);
  SB_BEHIND_WAIT(block_table);
  const int row = blockIdx.x;
  const T* pr = proj + (size_t)row * proj_width;
  if (q_rank > 0) {
    float sq = 0.f;
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x) {
      const float v = to_f<T>(pr[c]);
      sq += v * v;
    }
    sq = block_sum(sq, scratch);
    const float inv = 1.f / sqrtf(sq / (float)q_rank + eps);
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x)
      cq[(size_t)row * q_rank + c] = from_f<T>(to_f<T>(pr[c]) * inv * qg[c]);
  }
  if (!write) return;
  const int pos = tok_pos[row];
  const int page = block_table[(size_t)tok_slot[row] * table_stride + pos / SB_PAGE_TOKENS];
  T* dst = store + page_row(page, 0, pos % SB_PAGE_TOKENS, 1, rank + rot);
  const T* kv = pr + q_rank;
  float sq = 0.f;
  for (int c = threadIdx.x; c < rank; c += blockDim.x) {
    const float v = to_f<T>(kv[c]);
    sq += v * v;
  }
  sq = block_sum(sq, scratch);
  const float inv = 1.f / sqrtf(sq / (float)rank + eps);
  for (int c = threadIdx.x; c < rank; c += blockDim.x) dst[c] = from_f<T>(to_f<T>(kv[c]) * inv * kg[c]);
  const T* shared = kv + rank;
  for (int i = threadIdx.x; i < rot_dims / 2; i += blockDim.x) {
    const float a = to_f<T>(shared[2 * i]), b = to_f<T>(shared[2 * i + 1]);
    const float c = cos_t[(size_t)pos * table_width + i], s = sin_t[(size_t)pos * table_width + i];
    dst[rank + 2 * i] = from_f<T>(a * c - b * s);
    dst[rank + 2 * i + 1] = from_f<T>(b * c + a * s);
  }
  for (int c = rot_dims + threadIdx.x; c < rot; c += blockDim.x) dst[rank + c] = shared[c];
}

// q: [tokens, heads, dim + rot]; qa: [tokens, heads, rank + rot], whose first `rank` entries per head
// the caller fills; this files the turned last `rot` entries of q behind them.
template <typename T>
__global__ void latent_rotate_q_kernel(const T* __restrict__ q, T* __restrict__ qa, const float* __restrict__ cos_t,
                                       const float* __restrict__ sin_t, int table_width,
                                       const int* __restrict__ tok_pos, int heads, int dim, int rot, int rot_dims,
                                       int rank) {
  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(q);
  SB_BEHIND_WAIT(tok_pos);
  const int row = blockIdx.x;
  const int pos = tok_pos[row];
  const int half = rot_dims / 2, rest = rot - rot_dims;
  const int per_head = half + rest;
  for (int e = threadIdx.x; e < heads * per_head; e += blockDim.x) {
    const int h = e / per_head, i = e - h * per_head;
    const T* src = q + ((size_t)row * heads + h) * (dim + rot) + dim;
    T* dst = qa + ((size_t)row * heads + h) * (rank + rot) + rank;
    if (i < half) {
      const float a = to_f<T>(src[2 * i]), b = to_f<T>(src[2 * i + 1]);
      const float c = cos_t[(size_t)pos * table_width + i], s = sin_t[(size_t)pos * table_width + i];
      dst[2 * i] = from_f<T>(a * c - b * s);
      dst[2 * i + 1] = from_f<T>(b * c + a * s);
    } else {
      dst[rot_dims + i - half] = src[rot_dims + i - half];
    }
  }
}

// The plain kernel: one warp per (token, head), lanes over the entries of a row; NI = entries a lane.
template <typename T, int NI>
__global__ void latent_attention_kernel(const T* __restrict__ qa, T* __restrict__ out, const T* __restrict__ store,
                                        const int* __restrict__ block_table, int table_stride,
                                        const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
                                        int n_tokens, int heads, int rank, int rot, float scale, int window) {
  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(qa);
  SB_BEHIND_WAIT(store);
  SB_BEHIND_WAIT(tok_slot);
  SB_BEHIND_WAIT(tok_pos);
  SB_BEHIND_WAIT(block_table);
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= (long long)n_tokens * heads) return;
  const int token = (int)(warp / heads);
  const int width = rank + rot;
  const int pos = tok_pos[token];
  const int* pages = block_table + (size_t)tok_slot[token] * table_stride;
  const T* qr = qa + (size_t)warp * width;
  float qv[NI], acc[NI];
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int d = lane + 32 * i;
    qv[i] = d < width ? to_f<T>(qr[d]) * scale : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  int first = 0;
  if (window > 0 && pos - window + 1 > 0) first = pos - window + 1;
  for (int j0 = first; j0 <= pos; j0 += 4) {
    float s[4];
    float kvv[4][NI];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = j0 + u;
      s[u] = 0.f;
      if (j <= pos) {
        const T* kr = store + page_row(pages[j / SB_PAGE_TOKENS], 0, j % SB_PAGE_TOKENS, 1, width);
#pragma unroll
        for (int i = 0; i < NI; ++i) {
          const int d = lane + 32 * i;
          kvv[u][i] = d < width ? to_f<T>(kr[d]) : 0.f;
          s[u] += qv[i] * kvv[u][i];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) s[u] = warp_sum(s[u]);
    float m_new = m;
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (j0 + u <= pos) m_new = fmaxf(m_new, s[u]);
    const float alpha = expf(m - m_new);
    l *= alpha;
#pragma unroll
    for (int i = 0; i < NI; ++i) acc[i] *= alpha;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (j0 + u <= pos) {
        const float p = expf(s[u] - m_new);
        l += p;
#pragma unroll
        for (int i = 0; i < NI; ++i) acc[i] += p * kvv[u][i];
      }
    }
    m = m_new;
  }
  T* orow = out + (size_t)warp * rank;
  const float inv = 1.f / l;
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int d = lane + 32 * i;
    if (d < rank) orow[d] = from_f<T>(acc[i] * inv);
  }
}

template <typename T>
static int launch_attention(const void* qa, void* out, const void* store, const int* block_table, int table_stride,
                            const int* tok_slot, const int* tok_pos, int n_tokens, int heads, int rank, int rot,
                            float scale, int window, cudaStream_t s) {
  const long long warps = (long long)n_tokens * heads;
  const int threads = 128;
  const dim3 grid((unsigned)((warps * 32 + threads - 1) / threads));
  const int ni = (rank + rot + 31) / 32;
#define GO(N) return launch_dependent(latent_attention_kernel<T, N>, grid, dim3(threads), 0, s, (const T*)qa, (T*)out, \
    (const T*)store, block_table, table_stride, tok_slot, tok_pos, n_tokens, heads, rank, rot, scale, window)
  if (ni <= 2) GO(2);
  if (ni <= 4) GO(4);
  if (ni <= 8) GO(8);
  if (ni <= 12) GO(12);
  if (ni <= 20) GO(20);
#undef GO
  return -2;
}

extern "C" {

int sb_latent_max_row() { return 32 * 20; }

// proj: [n_tokens, proj_width], a row = [query latent (q_rank) | key/value latent (rank) | shared key
// part (rot)] (the query latent alone when write == 0).  cq: [n_tokens, q_rank].  store: one cache
// entry's pages [pages, 1, 64, rank + rot].  cos/sin: float [positions, table_width].
int sb_latent_prepare(int dtype, const void* proj, int proj_width, const float* qg, const float* kg, float eps,
                      const float* cos_t, const float* sin_t, int table_width, const int* tok_pos,
                      const int* tok_slot, const int* block_table, int table_stride, void* store, void* cq,
                      int n_tokens, int q_rank, int rank, int rot, int rot_dims, int write, cudaStream_t s) {
  if (n_tokens == 0) return 0;
  if (rot_dims % 2 || rot_dims > rot || rot_dims / 2 > table_width) return -2;
  if (proj_width < q_rank + (write ? rank + rot : 0)) return -2;
  if (dtype == 0)
    return launch_dependent(latent_prepare_kernel<float>, dim3(n_tokens), dim3(128), 0, s, (const float*)proj,
                            proj_width, qg, kg, eps, cos_t, sin_t, table_width, tok_pos, tok_slot, block_table,
                            table_stride, (float*)store, (float*)cq, q_rank, rank, rot, rot_dims, write);
  return launch_dependent(latent_prepare_kernel<bf16>, dim3(n_tokens), dim3(128), 0, s, (const bf16*)proj, proj_width,
                          qg, kg, eps, cos_t, sin_t, table_width, tok_pos, tok_slot, block_table, table_stride,
                          (bf16*)store, (bf16*)cq, q_rank, rank, rot, rot_dims, write);
}

int sb_latent_rotate_q(int dtype, const void* q, void* qa, const float* cos_t, const float* sin_t, int table_width,
                       const int* tok_pos, int n_tokens, int heads, int dim, int rot, int rot_dims, int rank,
                       cudaStream_t s) {
  if (n_tokens == 0 || rot == 0) return 0;
  if (rot_dims % 2 || rot_dims > rot || rot_dims / 2 > table_width) return -2;
  if (dtype == 0)
    return launch_dependent(latent_rotate_q_kernel<float>, dim3(n_tokens), dim3(128), 0, s, (const float*)q,
                            (float*)qa, cos_t, sin_t, table_width, tok_pos, heads, dim, rot, rot_dims, rank);
  return launch_dependent(latent_rotate_q_kernel<bf16>, dim3(n_tokens), dim3(128), 0, s, (const bf16*)q, (bf16*)qa,
                          cos_t, sin_t, table_width, tok_pos, heads, dim, rot, rot_dims, rank);
}

// qa: [n_tokens, heads, rank + rot]; out: [n_tokens, heads, rank]; store as above.
int sb_latent_attention(int dtype, const void* qa, void* out, const void* store, const int* block_table,
                        int table_stride, const int* tok_slot, const int* tok_pos, int n_tokens, int heads, int rank,
                        int rot, float scale, int window, cudaStream_t s) {
  if (n_tokens == 0) return 0;
  if (dtype == 0)
    return launch_attention<float>(qa, out, store, block_table, table_stride, tok_slot, tok_pos, n_tokens, heads,
                                   rank, rot, scale, window, s);
  return launch_attention<bf16>(qa, out, store, block_table, table_stride, tok_slot, tok_pos, n_tokens, heads, rank,
                                rot, scale, window, s);
}

}  // extern "C"
