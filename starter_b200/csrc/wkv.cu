// A linear recurrence with a matrix state per head and a decay that depends on the token (the time
// mixing of the RWKV family), over packed sequences, with the state kept per cache slot.
//
// Per head, with r, k, v, w of `dim` entries each for token t and a bonus vector u:
//
//     o_t[j] = sum_i r_t[i] * (S[i][j] + u[i] * k_t[i] * v_t[j])          S before this token
//     S[i][j] <- w_t[i] * S[i][j] + k_t[i] * v_t[j]
//     w_t[i]  = exp(-exp(x_t[i] + w0[i]))                                  x: the decay projection
//
// then the head's o is divided by its root mean square, multiplied by a gain and by silu(g).  The
// state, the decay and its exponentials, the sums and the head norm are float whatever the working
// type; r, k, v and g arrive in the working type (they are projections).
//
// The same kernel serves a whole prompt, a later portion and a single token: a block owns one
// (sequence of the step, head), reads S from the sequence's slot, walks the tokens the sequence brings
// and writes S back.  A slot's state is `state_stride` floats: the previous token's mixer input
// (`width` floats, what token_shift reads for a portion's first token) and then S as
// [heads][dim (j)][dim (i)].
#include "common.cuh"

#define WKV_CHUNK 16
#define WKV_PREFETCH 32

// out[s][t][c] = h[t][c] + (prev[t][c] - h[t][c]) * mu[s][c] for s < n_mix; prev is the row before in
// the same sequence, or what the slot's state holds when the row is the first its sequence brings.
template <typename T>
__global__ void token_shift_kernel(const T* __restrict__ h, const float* __restrict__ state, size_t state_stride,
                                   const float* __restrict__ mu, T* __restrict__ out,
                                   const int* __restrict__ tok_slot, int n_tokens, int width, int n_mix) {
  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(h);
  SB_BEHIND_WAIT(state);
  SB_BEHIND_WAIT(tok_slot);
  const int row = blockIdx.x;
  const int slot = tok_slot[row];
  const bool first = row == 0 || tok_slot[row - 1] != slot;
  const T* cur = h + (size_t)row * width;
  const T* before = h + (size_t)(row - 1) * width;
  const float* held = state + (size_t)slot * state_stride;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float x = to_f<T>(cur[c]);
    const float p = first ? held[c] : to_f<T>(before[c]);
    for (int s = 0; s < n_mix; ++s)
      out[((size_t)s * n_tokens + row) * width + c] = from_f<T>(x + (p - x) * mu[(size_t)s * width + c]);
  }
}

// Thread (j, p) holds S[i][j] for i = p, p + P, ...: KPT values.  P is a power of two (at most 32),
// the P threads of a j are neighbouring lanes and sum their parts of o[j] by shuffles.
template <typename T, int KPT>
__global__ void __launch_bounds__(KPT > 32 ? 1024 : 512)
wkv_scan_kernel(const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v,
                const float* __restrict__ x_decay, const float* __restrict__ w0, const float* __restrict__ u,
                const T* __restrict__ g, const float* __restrict__ gain, float* __restrict__ state,
                size_t state_stride, int state_offset, const T* __restrict__ h, int width, T* __restrict__ out,
                const int* __restrict__ seq_slot, const int* __restrict__ seq_q_start,
                const int* __restrict__ seq_q_len, int heads, int D, int P, float eps) {
  extern __shared__ float smem[];
  const int tid = threadIdx.x, nt = blockDim.x;
  const int seq = blockIdx.x, head = blockIdx.y;
  const int j = tid / P, p = tid % P;
  const bool live = j < D;
  const int hd = heads * D;
  // [2][4][CHUNK][D] inputs (r, k, w, v) and [CHUNK][D] outputs
  float* in_buf = smem;
  float* o_buf = smem + 2 * 4 * WKV_CHUNK * D;
  float uu[KPT];
#pragma unroll
  for (int m = 0; m < KPT; ++m) {
    const int i = p + P * m;
    uu[m] = (live && i < D) ? u[head * D + i] : 0.f;
  }
  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(r); SB_BEHIND_WAIT(k); SB_BEHIND_WAIT(v); SB_BEHIND_WAIT(x_decay); SB_BEHIND_WAIT(g);
  SB_BEHIND_WAIT(state); SB_BEHIND_WAIT(h);
  SB_BEHIND_WAIT(seq_slot); SB_BEHIND_WAIT(seq_q_start); SB_BEHIND_WAIT(seq_q_len);
  const int slot = seq_slot[seq], q_start = seq_q_start[seq], q_len = seq_q_len[seq];
  float* held = state + (size_t)slot * state_stride;
  float* S_mem = held + state_offset + ((size_t)head * D + (live ? j : 0)) * D;
  float S[KPT];
#pragma unroll
  for (int m = 0; m < KPT; ++m) {
    const int i = p + P * m;
    S[m] = (live && i < D) ? S_mem[i] : 0.f;
  }
  const int per_chunk = 4 * WKV_CHUNK * D;
  const int n_chunks = (q_len + WKV_CHUNK - 1) / WKV_CHUNK;
  float pre[WKV_PREFETCH];

  auto fetch = [&](int chunk) {
#pragma unroll
    for (int n = 0; n < WKV_PREFETCH; ++n) {
      const int e = tid + n * nt;
      pre[n] = 0.f;
      if (e < per_chunk) {
        const int a = e / (WKV_CHUNK * D), rem = e - a * (WKV_CHUNK * D);
        const int tt = rem / D, d = rem - tt * D;
        const int t = chunk * WKV_CHUNK + tt;
        if (t < q_len) {
          const size_t at = (size_t)(q_start + t) * hd + head * D + d;
          pre[n] = a == 0 ? to_f<T>(r[at]) : a == 1 ? to_f<T>(k[at]) : a == 2 ? x_decay[at] : to_f<T>(v[at]);
        }
      }
    }
  };
  auto stash = [&](int buf) {
    float* dst = in_buf + (size_t)buf * per_chunk;
#pragma unroll
    for (int n = 0; n < WKV_PREFETCH; ++n) {
      const int e = tid + n * nt;
      if (e < per_chunk) {
        const int a = e / (WKV_CHUNK * D), rem = e - a * (WKV_CHUNK * D);
        float val = pre[n];
        if (a == 2) val = expf(-expf(val + w0[head * D + (rem % D)]));
        dst[e] = val;
      }
    }
  };

  fetch(0);
  stash(0);
  __syncthreads();
  for (int c = 0; c < n_chunks; ++c) {
    const int buf = c & 1;
    if (c + 1 < n_chunks) fetch(c + 1);
    const float* rs = in_buf + (size_t)buf * per_chunk;
    const float* ks = rs + WKV_CHUNK * D;
    const float* ws = ks + WKV_CHUNK * D;
    const float* vs = ws + WKV_CHUNK * D;
    const int here = min(WKV_CHUNK, q_len - c * WKV_CHUNK);
    for (int tt = 0; tt < here; ++tt) {
      const float vj = live ? vs[tt * D + j] : 0.f;
      float acc = 0.f;
#pragma unroll
      for (int m = 0; m < KPT; ++m) {
        const int i = p + P * m;
        if (i < D) {
          const float kv = ks[tt * D + i] * vj;
          acc += rs[tt * D + i] * (S[m] + uu[m] * kv);
          S[m] = ws[tt * D + i] * S[m] + kv;
        }
      }
      for (int o = P >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (live && p == 0) o_buf[tt * D + j] = acc;
    }
    __syncthreads();
    // the head norm, the gain and the gate for this chunk's tokens: a warp a token
    for (int tt = tid >> 5; tt < here; tt += nt >> 5) {
      const int lane = tid & 31;
      float sq = 0.f;
      for (int d = lane; d < D; d += 32) sq += o_buf[tt * D + d] * o_buf[tt * D + d];
      sq = warp_sum(sq);
      const float inv = 1.f / sqrtf(sq / (float)D + eps);
      const size_t at = (size_t)(q_start + c * WKV_CHUNK + tt) * hd + head * D;
      for (int d = lane; d < D; d += 32) {
        const float gv = to_f<T>(g[at + d]);
        out[at + d] = from_f<T>(o_buf[tt * D + d] * inv * gain[head * D + d] * (gv / (1.f + expf(-gv))));
      }
    }
    if (c + 1 < n_chunks) stash(buf ^ 1);
    __syncthreads();
  }
#pragma unroll
  for (int m = 0; m < KPT; ++m) {
    const int i = p + P * m;
    if (live && i < D) S_mem[i] = S[m];
  }
  if (head == 0) {
    // the sequence's last mixer input: what the next portion's first token is shifted with
    const T* last = h + (size_t)(q_start + q_len - 1) * width;
    for (int c = tid; c < width; c += nt) held[c] = to_f<T>(last[c]);
  }
}

template <typename T>
static int launch_scan(const void* r, const void* k, const void* v, const float* x_decay, const float* w0,
                       const float* u, const void* g, const float* gain, float* state, size_t state_stride,
                       int state_offset, const void* h, int width, void* out, const int* seq_slot,
                       const int* seq_q_start, const int* seq_q_len, int n_seqs, int heads, int D, float eps,
                       cudaStream_t s) {
  const int kpt = D <= 64 ? 8 : D <= 128 ? 32 : 64;
  int P = 1;
  while (P * kpt < D) P *= 2;
  int threads = (D * P + 31) / 32 * 32;
  if (P > 32 || threads > (kpt > 32 ? 1024 : 512) || 4 * WKV_CHUNK * D > WKV_PREFETCH * threads) return -2;
  const size_t smem = (size_t)(2 * 4 + 1) * WKV_CHUNK * D * sizeof(float);
  const dim3 grid(n_seqs, heads);
  if (kpt == 8) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(wkv_scan_kernel<T, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_dependent(wkv_scan_kernel<T, 8>, grid, dim3(threads), smem, s, (const T*)r, (const T*)k, (const T*)v,
                            x_decay, w0, u, (const T*)g, gain, state, state_stride, state_offset, (const T*)h, width,
                            (T*)out, seq_slot, seq_q_start, seq_q_len, heads, D, P, eps);
  }
  if (kpt == 64) {
    // heads of up to 256 channels: 64 state values a thread at 1,024 threads, which the compiler keeps
    // partly in local memory; correct, and slower than the sizes above
    cudaFuncSetAttribute(wkv_scan_kernel<T, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_dependent(wkv_scan_kernel<T, 64>, grid, dim3(threads), smem, s, (const T*)r, (const T*)k, (const T*)v,
                            x_decay, w0, u, (const T*)g, gain, state, state_stride, state_offset, (const T*)h, width,
                            (T*)out, seq_slot, seq_q_start, seq_q_len, heads, D, P, eps);
  }
  if (smem > 48 * 1024) cudaFuncSetAttribute(wkv_scan_kernel<T, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return launch_dependent(wkv_scan_kernel<T, 32>, grid, dim3(threads), smem, s, (const T*)r, (const T*)k, (const T*)v,
                          x_decay, w0, u, (const T*)g, gain, state, state_stride, state_offset, (const T*)h, width,
                          (T*)out, seq_slot, seq_q_start, seq_q_len, heads, D, P, eps);
}

extern "C" {

int sb_wkv_max_dim() { return 256; }

// h: [n_tokens, width]; state: float [slots, state_stride], a slot's first `width` floats hold the
// mixer input of the last token before this step; mu: float [n_mix, width]; out: [n_mix, n_tokens, width].
int sb_token_shift(int dtype, const void* h, const float* state, long long state_stride, const float* mu,
                   void* out, const int* tok_slot, int n_tokens, int width, int n_mix, cudaStream_t s) {
  if (n_tokens == 0) return 0;
  const int threads = width >= 1024 ? 256 : 128;
  if (dtype == 0)
    return launch_dependent(token_shift_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, (const float*)h, state,
                            (size_t)state_stride, mu, (float*)out, tok_slot, n_tokens, width, n_mix);
  return launch_dependent(token_shift_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, s, (const bf16*)h, state,
                          (size_t)state_stride, mu, (bf16*)out, tok_slot, n_tokens, width, n_mix);
}

// r, k, v, g, out: [n_tokens, heads * dim] of the working type; x_decay: float, same shape; w0, gain:
// float [heads * dim]; u: float [heads, dim].  The state of a slot: see the head of this file
// (state_offset = where S starts inside a slot's floats).
int sb_wkv_scan(int dtype, const void* r, const void* k, const void* v, const float* x_decay, const float* w0,
                const float* u, const void* g, const float* gain, float* state, long long state_stride,
                int state_offset, const void* h, int width, void* out, const int* seq_slot, const int* seq_q_start,
                const int* seq_q_len, int n_seqs, int heads, int dim, float eps, cudaStream_t s) {
  if (n_seqs == 0) return 0;
  if (dim < 1 || dim > 256 || heads < 1) return -2;
  if (dtype == 0)
    return launch_scan<float>(r, k, v, x_decay, w0, u, g, gain, state, (size_t)state_stride, state_offset, h, width,
                              out, seq_slot, seq_q_start, seq_q_len, n_seqs, heads, dim, eps, s);
  return launch_scan<bf16>(r, k, v, x_decay, w0, u, g, gain, state, (size_t)state_stride, state_offset, h, width,
                           out, seq_slot, seq_q_start, seq_q_len, n_seqs, heads, dim, eps, s);
}

}  // extern "C"
