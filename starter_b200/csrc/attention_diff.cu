// Differential attention over the paged cache: two softmax maps per head over the same values.
//
// A query head has two query vectors q1, q2 (`dim` each, stored [q1 | q2]); its key/value head has
// two key vectors per token, stored the same way, and ONE value vector of `v_dim`.  With
//     a_m = softmax(scale * q_m . k_m over the visible keys) . v        (m = 1, 2)
// the head's output is
//     o = a_1 - lambda * a_2,   o <- o / sqrt(mean(o^2) + eps) * out_scale,   o <- o * sigmoid(gate)
// (lambda one number per layer, the unit norm over the head's v_dim values, the gate optional).
// Visibility is by absolute position: key j is seen by the query at p iff j <= p (and, with a window
// w, j > p - w).  The cache keeps a token's keys as one row of 2 * dim per key/value head and its
// values as one row of v_dim: [pages][kv_heads][64][2 * dim] and [pages][kv_heads][64][v_dim].
// Scores, softmax weights, both accumulators, lambda, the norm and the gate are float.
//
// Kernels here:
//   diff_prepare     adds the projection biases, scales the queries by their temperature
//                    1 + coef * ln(floor((p + 1) / every) + 1), files keys and values at each token's place
//   diff_attention   one block per (token, head); its warps share the keys, merge, then finish the head
//                    (any sizes, both types: single tokens, the 32-bit path, short chunks)
// The bfloat16 tensor-core kernels for prompts and for single tokens are in attention_diff_prefill.cu.
#include "common.cuh"

#define SB_DIFF_MAX_I 8   // 2 * dim <= 256 and v_dim <= 256

// ------------------------------------------------------------------------------------ prepare

// proj row: [q (heads * qk) | gate (heads * v_dim, untouched here) | k (kv_heads * qk) | v (kv_heads * v_dim)],
// the last two only with write_cache.  bias: float, same layout, or null.
template <typename T>
__global__ void diff_prepare_kernel(const T* __restrict__ proj, int proj_stride, const float* __restrict__ bias,
                                    T* __restrict__ q_out, const int* __restrict__ tok_pos,
                                    const int* __restrict__ tok_slot, const int* __restrict__ block_table,
                                    int table_stride, T* __restrict__ k_store, T* __restrict__ v_store,
                                    int heads, int kv_heads, int qk, int v_dim, int gate_width, float temp_coef,
                                    int temp_every, int write_cache) {
  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(proj);
  SB_BEHIND_WAIT(tok_pos);
  SB_BEHIND_WAIT(tok_slot);
  const int token = blockIdx.x;
  const int pos = tok_pos[token];
  const T* row = proj + (size_t)token * proj_stride;
  const int q_w = heads * qk;
  float temp = 1.f;
  if (temp_every > 0) temp = 1.f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.f);
  T* qr = q_out + (size_t)token * q_w;
  for (int c = threadIdx.x; c < q_w; c += blockDim.x) {
    float v = to_f<T>(row[c]);
    if (bias) v = rnd<T>(v + bias[c]);
    qr[c] = from_f<T>(v * temp);
  }
  if (!write_cache) return;
  const int page = block_table[(size_t)tok_slot[token] * table_stride + pos / SB_PAGE_TOKENS];
  const int off = pos % SB_PAGE_TOKENS;
  const int k0 = q_w + gate_width, k_w = kv_heads * qk, v_w = kv_heads * v_dim;
  for (int c = threadIdx.x; c < k_w; c += blockDim.x) {
    float v = to_f<T>(row[k0 + c]);
    if (bias) v += bias[k0 + c];
    const int h = c / qk;
    k_store[page_row(page, h, off, kv_heads, qk) + (c - h * qk)] = from_f<T>(v);
  }
  for (int c = threadIdx.x; c < v_w; c += blockDim.x) {
    float v = to_f<T>(row[k0 + k_w + c]);
    if (bias) v += bias[k0 + k_w + c];
    const int h = c / v_dim;
    v_store[page_row(page, h, off, kv_heads, v_dim) + (c - h * v_dim)] = from_f<T>(v);
  }
}

// The same with eight consecutive columns a thread (16-byte accesses for bfloat16) and a row cut into
// pieces (blockIdx.y): needs 2 * dim, v_dim, the gate's width and the row stride to be multiples of 8
// and 16-byte aligned bases.
template <typename T> __device__ __forceinline__ void load8(const T* p, float* out) {
  if (sizeof(T) == 2) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = to_f<T>(e[i]);
  } else {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w; out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
  }
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float* v) {
  if (sizeof(T) == 2) {
    uint4 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) e[i] = from_f<T>(v[i]);
    *reinterpret_cast<uint4*>(p) = raw;
  } else {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
}

template <typename T>
__global__ void diff_prepare_vec_kernel(const T* __restrict__ proj, int proj_stride, const float* __restrict__ bias,
                                        T* __restrict__ q_out, const int* __restrict__ tok_pos,
                                        const int* __restrict__ tok_slot, const int* __restrict__ block_table,
                                        int table_stride, T* __restrict__ k_store, T* __restrict__ v_store,
                                        int heads, int kv_heads, int qk, int v_dim, int gate_width, float temp_coef,
                                        int temp_every, int write_cache) {
  const int q_w = heads * qk, k_w = kv_heads * qk, v_w = kv_heads * v_dim;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;      // column among [q | k | v]
  const int src = c < q_w ? c : c + gate_width;                   // column of the stacked row
  float bv[8];
  const bool live = c < q_w + (write_cache ? k_w + v_w : 0);
  if (live && bias) load8<float>(bias + src, bv);
  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(proj);
  SB_BEHIND_WAIT(tok_pos);
  SB_BEHIND_WAIT(tok_slot);
  if (!live) return;
  const int token = blockIdx.x;
  const int pos = tok_pos[token];
  float v[8];
  load8<T>(proj + (size_t)token * proj_stride + src, v);
  if (c < q_w) {
    float temp = 1.f;
    if (temp_every > 0) temp = 1.f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.f);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = (bias ? rnd<T>(v[i] + bv[i]) : v[i]) * temp;
    store8<T>(q_out + (size_t)token * q_w + c, v);
    return;
  }
  if (bias) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] += bv[i];
  }
  const int page = block_table[(size_t)tok_slot[token] * table_stride + pos / SB_PAGE_TOKENS];
  const int off = pos % SB_PAGE_TOKENS;
  if (c < q_w + k_w) {
    const int cc = c - q_w, h = cc / qk;
    store8<T>(k_store + page_row(page, h, off, kv_heads, qk) + (cc - h * qk), v);
  } else {
    const int cc = c - q_w - k_w, h = cc / v_dim;
    store8<T>(v_store + page_row(page, h, off, kv_heads, v_dim) + (cc - h * v_dim), v);
  }
}

// ------------------------------------------------------------------------------------ general kernel

struct DiffTail {
  float lambda, out_scale, eps;
};

// One block per (token, head).  Warp w takes the keys first + 4 * (w + warps * i) .. + 3; the warps'
// partial results (maximum, sum, accumulator, per map) meet in shared memory.
template <typename T>
__global__ void diff_attention_kernel(const T* __restrict__ q, const T* __restrict__ gate, int gate_stride,
                                      T* __restrict__ out, const T* __restrict__ k_store,
                                      const T* __restrict__ v_store, const int* __restrict__ block_table,
                                      int table_stride, const int* __restrict__ tok_slot,
                                      const int* __restrict__ tok_pos, int heads, int kv_heads, int dim,
                                      int v_dim, float scale, int window, DiffTail tail) {
  extern __shared__ float smem[];          // [warps][2][2 + v_dim] + 33
  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(q);
  SB_BEHIND_WAIT(gate);
  SB_BEHIND_WAIT(tok_slot);
  SB_BEHIND_WAIT(tok_pos);
  SB_BEHIND_WAIT(k_store);
  SB_BEHIND_WAIT(v_store);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int token = blockIdx.x / heads;
  const int h = blockIdx.x - token * heads;
  const int kvh = h / (heads / kv_heads);
  const int qk = 2 * dim;
  const int pos = tok_pos[token];
  const int* pages = block_table + (size_t)tok_slot[token] * table_stride;
  const T* qr = q + ((size_t)token * heads + h) * qk;

  float qv[SB_DIFF_MAX_I], acc1[SB_DIFF_MAX_I], acc2[SB_DIFF_MAX_I];
#pragma unroll
  for (int i = 0; i < SB_DIFF_MAX_I; ++i) {
    const int d = lane + 32 * i;
    qv[i] = d < qk ? to_f<T>(qr[d]) * scale : 0.f;
    acc1[i] = acc2[i] = 0.f;
  }
  float m1 = -INFINITY, l1 = 0.f, m2 = -INFINITY, l2 = 0.f;
  int first = 0;
  if (window > 0 && pos - window + 1 > 0) first = pos - window + 1;

  for (int j0 = first + 4 * warp; j0 <= pos; j0 += 4 * warps) {
    float s1[4], s2[4];
    const T* vrow[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = j0 + u;
      s1[u] = s2[u] = 0.f;
      vrow[u] = nullptr;
      if (j <= pos) {
        const int page = pages[j / SB_PAGE_TOKENS];
        const T* kr = k_store + page_row(page, kvh, j % SB_PAGE_TOKENS, kv_heads, qk);
        vrow[u] = v_store + page_row(page, kvh, j % SB_PAGE_TOKENS, kv_heads, v_dim);
#pragma unroll
        for (int i = 0; i < SB_DIFF_MAX_I; ++i) {
          const int d = lane + 32 * i;
          if (d < qk) {
            const float p = qv[i] * to_f<T>(kr[d]);
            if (d < dim) s1[u] += p; else s2[u] += p;
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) { s1[u] = warp_sum(s1[u]); s2[u] = warp_sum(s2[u]); }
    float n1 = m1, n2 = m2;
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (j0 + u <= pos) { n1 = fmaxf(n1, s1[u]); n2 = fmaxf(n2, s2[u]); }
    const float r1 = expf(m1 - n1), r2 = expf(m2 - n2);
    l1 *= r1; l2 *= r2;
#pragma unroll
    for (int i = 0; i < SB_DIFF_MAX_I; ++i) { acc1[i] *= r1; acc2[i] *= r2; }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (j0 + u <= pos) {
        const float p1 = expf(s1[u] - n1), p2 = expf(s2[u] - n2);
        l1 += p1; l2 += p2;
#pragma unroll
        for (int i = 0; i < SB_DIFF_MAX_I; ++i) {
          const int d = lane + 32 * i;
          if (d < v_dim) {
            const float v = to_f<T>(vrow[u][d]);
            acc1[i] += p1 * v;
            acc2[i] += p2 * v;
          }
        }
      }
    }
    m1 = n1; m2 = n2;
  }

  const int per = 2 + v_dim;
  float* mine = smem + (size_t)warp * 2 * per;
  if (lane == 0) { mine[0] = m1; mine[1] = l1; mine[per] = m2; mine[per + 1] = l2; }
#pragma unroll
  for (int i = 0; i < SB_DIFF_MAX_I; ++i) {
    const int d = lane + 32 * i;
    if (d < v_dim) { mine[2 + d] = acc1[i]; mine[per + 2 + d] = acc2[i]; }
  }
  __syncthreads();
  float* scratch = smem + (size_t)warps * 2 * per;
  // every thread finishes the columns it owns (v_dim may exceed the block: loop), twice: once for the
  // sum of squares, once to write
  float big1 = -INFINITY, big2 = -INFINITY;
  for (int w = 0; w < warps; ++w) {
    big1 = fmaxf(big1, smem[(size_t)w * 2 * per]);
    big2 = fmaxf(big2, smem[(size_t)w * 2 * per + per]);
  }
  float den1 = 0.f, den2 = 0.f;
  for (int w = 0; w < warps; ++w) {
    den1 += smem[(size_t)w * 2 * per + 1] * expf(smem[(size_t)w * 2 * per] - big1);
    den2 += smem[(size_t)w * 2 * per + per + 1] * expf(smem[(size_t)w * 2 * per + per] - big2);
  }
  float ss = 0.f;
  for (int c = threadIdx.x; c < v_dim; c += blockDim.x) {
    float a1 = 0.f, a2 = 0.f;
    for (int w = 0; w < warps; ++w) {
      a1 += smem[(size_t)w * 2 * per + 2 + c] * expf(smem[(size_t)w * 2 * per] - big1);
      a2 += smem[(size_t)w * 2 * per + per + 2 + c] * expf(smem[(size_t)w * 2 * per + per] - big2);
    }
    const float o = a1 / den1 - tail.lambda * (a2 / den2);
    ss += o * o;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)v_dim + tail.eps) * tail.out_scale;
  T* orow = out + ((size_t)token * heads + h) * v_dim;
  const T* grow = gate ? gate + (size_t)token * gate_stride + (size_t)h * v_dim : nullptr;
  for (int c = threadIdx.x; c < v_dim; c += blockDim.x) {
    float a1 = 0.f, a2 = 0.f;
    for (int w = 0; w < warps; ++w) {
      a1 += smem[(size_t)w * 2 * per + 2 + c] * expf(smem[(size_t)w * 2 * per] - big1);
      a2 += smem[(size_t)w * 2 * per + per + 2 + c] * expf(smem[(size_t)w * 2 * per + per] - big2);
    }
    float o = (a1 / den1 - tail.lambda * (a2 / den2)) * inv;
    if (grow) o *= 1.f / (1.f + expf(-to_f<T>(grow[c])));
    orow[c] = from_f<T>(o);
  }
}

extern "C" {

int sb_diff_prepare(int dtype, const void* proj, int proj_stride, const float* bias, void* q_out,
                    const int* tok_pos, const int* tok_slot, const int* block_table, int table_stride,
                    void* k_store, void* v_store, int n_tokens, int heads, int kv_heads, int dim, int v_dim,
                    int gate_width, float temp_coef, int temp_every, int write_cache, cudaStream_t s) {
  if (n_tokens == 0) return 0;
  const int threads = 128;
  const int qk = 2 * dim;
  const uintptr_t all = (uintptr_t)proj | (uintptr_t)bias | (uintptr_t)q_out | (uintptr_t)k_store | (uintptr_t)v_store;
  if (qk % 8 == 0 && v_dim % 8 == 0 && gate_width % 8 == 0 && proj_stride % 8 == 0 && (all & 15) == 0) {
    const int cols = heads * qk + (write_cache ? kv_heads * (qk + v_dim) : 0);
    const dim3 grid(n_tokens, (cols / 8 + threads - 1) / threads);
    if (dtype == 0)
      return launch_dependent(diff_prepare_vec_kernel<float>, grid, dim3(threads), 0, s, (const float*)proj,
                              proj_stride, bias, (float*)q_out, tok_pos, tok_slot, block_table, table_stride,
                              (float*)k_store, (float*)v_store, heads, kv_heads, qk, v_dim, gate_width,
                              temp_coef, temp_every, write_cache);
    return launch_dependent(diff_prepare_vec_kernel<bf16>, grid, dim3(threads), 0, s, (const bf16*)proj,
                            proj_stride, bias, (bf16*)q_out, tok_pos, tok_slot, block_table, table_stride,
                            (bf16*)k_store, (bf16*)v_store, heads, kv_heads, qk, v_dim, gate_width,
                            temp_coef, temp_every, write_cache);
  }
  if (dtype == 0)
    return launch_dependent(diff_prepare_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, (const float*)proj,
                            proj_stride, bias, (float*)q_out, tok_pos, tok_slot, block_table, table_stride,
                            (float*)k_store, (float*)v_store, heads, kv_heads, 2 * dim, v_dim, gate_width,
                            temp_coef, temp_every, write_cache);
  return launch_dependent(diff_prepare_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, s, (const bf16*)proj,
                          proj_stride, bias, (bf16*)q_out, tok_pos, tok_slot, block_table, table_stride,
                          (bf16*)k_store, (bf16*)v_store, heads, kv_heads, 2 * dim, v_dim, gate_width,
                          temp_coef, temp_every, write_cache);
}

// q [n_tokens, heads * 2 * dim]; gate null or rows of `gate_stride` elements whose first heads * v_dim
// are the gate's pre-activations; out [n_tokens, heads * v_dim].  warps: 1..16 per (token, head).
int sb_diff_attention(int dtype, const void* q, const void* gate, int gate_stride, void* out, const void* k_store,
                      const void* v_store, const int* block_table, int table_stride, const int* tok_slot,
                      const int* tok_pos, int n_tokens, int heads, int kv_heads, int dim, int v_dim, float scale,
                      int window, float lambda, float out_scale, float eps, int warps, cudaStream_t s) {
  if (2 * dim > 32 * SB_DIFF_MAX_I || v_dim > 32 * SB_DIFF_MAX_I || kv_heads <= 0 || heads % kv_heads) return -2;
  if (warps < 1 || warps > 16) return -2;
  if (n_tokens == 0) return 0;
  const long long blocks = (long long)n_tokens * heads;
  if (blocks > 0x7fffffffLL) return -2;
  const size_t smem = ((size_t)warps * 2 * (2 + v_dim) + 33) * sizeof(float);
  DiffTail tail = {lambda, out_scale, eps};
  if (dtype == 0)
    return launch_dependent(diff_attention_kernel<float>, dim3((unsigned)blocks), dim3(32 * warps), smem, s,
                            (const float*)q, (const float*)gate, gate_stride, (float*)out, (const float*)k_store,
                            (const float*)v_store, block_table, table_stride, tok_slot, tok_pos, heads, kv_heads,
                            dim, v_dim, scale, window, tail);
  return launch_dependent(diff_attention_kernel<bf16>, dim3((unsigned)blocks), dim3(32 * warps), smem, s,
                          (const bf16*)q, (const bf16*)gate, gate_stride, (bf16*)out, (const bf16*)k_store,
                          (const bf16*)v_store, block_table, table_stride, tok_slot, tok_pos, heads, kv_heads,
                          dim, v_dim, scale, window, tail);
}

}  // extern "C"
