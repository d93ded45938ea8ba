// Several residual streams per token (hyper-connections) and the Dynamic Tanh norm.
//
// A model with hyper-connections keeps S copies x_1..x_S of the residual stream per token, as
// float [tokens][S][hidden] (the residual is a 32-bit sum whatever the working type).  Around a
// sublayer with the vectors `in` [S], `out` [S] and the matrix `mix` [S][S] (indexed [from][to]):
//
//     u    = sum_s in[s] * x_s                       the sublayer's input, before its norm
//     y    = sublayer(norm(u))
//     x_t <- sum_s mix[s][t] * x_s + out[t] * y      every t from the x before the update
//
// The update that closes one sublayer and the read that opens the next touch the same S rows, so
// they are ONE kernel here (as the residual sum and the norm after it are one kernel in the
// single-stream models): hyper_step applies the pending update of the previous sublayer in place,
// forms u for the next one and norms it.  With `rows` it does the same for selected rows without
// writing back, and with in == null it forms the plain sum of the streams: that closes the model.
//
// Dynamic Tanh: y = tanh(alpha * x) * w + b with a scalar alpha; no mean, no variance.
#include "common.cuh"

#define SB_MAX_STREAMS 8

template <typename T>
__global__ void embed_streams_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                                     float* __restrict__ out, int hidden, int vocab, int streams, int* status) {
  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(tokens);
  const int row = blockIdx.x;
  int tok = tokens[row];
  const bool bad = tok < 0 || tok >= vocab;
  if (bad) {
    if (threadIdx.x == 0 && status) atomicOr(status, 1);
    tok = 0;
  }
  const T* src = table + (size_t)tok * hidden;
  float* dst = out + (size_t)row * streams * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float v = bad ? 0.f : to_f<T>(src[c]);
    for (int s = 0; s < streams; ++s) dst[(size_t)s * hidden + c] = v;
  }
}

// V consecutive values of T as floats and back (V = 4: one 8- or 16-byte access; V = 1: any address).
template <typename T, int V> __device__ __forceinline__ void load_v(const T* p, float* out) {
  if (V == 4 && sizeof(T) == 4) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  } else if (V == 4) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) out[i] = to_f<T>(e[i]);
  } else {
    out[0] = to_f<T>(p[0]);
  }
}
template <typename T, int V> __device__ __forceinline__ void store_v(T* p, const float* v) {
  if (V == 4 && sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  } else if (V == 4) {
    uint2 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) e[i] = from_f<T>(v[i]);
    *reinterpret_cast<uint2*>(p) = raw;
  } else {
    p[0] = from_f<T>(v[0]);
  }
}

// norm_kind 0: normed = u (rounded to T); 1: Dynamic Tanh of u.  Nothing here sums over a row, so a row
// is cut into pieces of blockDim * V columns (blockIdx.y) and a thread owns V consecutive columns.
template <typename T, int S, int V>
__global__ void hyper_step_kernel(float* __restrict__ streams, const T* __restrict__ y,
                                  const float* __restrict__ y_bias, const float* __restrict__ mix_prev,
                                  const float* __restrict__ out_prev, const float* __restrict__ in_next,
                                  int norm_kind, const float* __restrict__ alpha_p,
                                  const float* __restrict__ w, const float* __restrict__ b,
                                  T* __restrict__ normed, const int* __restrict__ rows, int hidden) {
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
  float mix[S * S], outw[S], inw[S];
#pragma unroll
  for (int i = 0; i < S * S; ++i) mix[i] = y ? mix_prev[i] : 0.f;
#pragma unroll
  for (int i = 0; i < S; ++i) {
    outw[i] = y ? out_prev[i] : 0.f;
    inw[i] = in_next ? in_next[i] : 1.f;
  }
  const float alpha = norm_kind == 1 ? alpha_p[0] : 0.f;
  float wv[V], bv[V], biasv[V];
  if (c < hidden) {
    if (norm_kind == 1) { load_v<float, V>(w + c, wv); load_v<float, V>(b + c, bv); }
    if (y && y_bias) load_v<float, V>(y_bias + c, biasv);
  }
  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(y);
  SB_BEHIND_WAIT(rows);
  if (c >= hidden) return;
  const int out_row = blockIdx.x;
  const int in_row = rows ? rows[out_row] : out_row;
  float* xr = streams + (size_t)in_row * S * hidden + c;
  float x[S][V];
#pragma unroll
  for (int s = 0; s < S; ++s) load_v<float, V>(xr + (size_t)s * hidden, x[s]);
  if (y) {
    float yv[V];
    load_v<T, V>(y + (size_t)in_row * hidden + c, yv);
    if (y_bias) {
#pragma unroll
      for (int i = 0; i < V; ++i) yv[i] += biasv[i];
    }
    float nx[S][V];
#pragma unroll
    for (int t = 0; t < S; ++t) {
#pragma unroll
      for (int i = 0; i < V; ++i) {
        float a = 0.f;
#pragma unroll
        for (int s = 0; s < S; ++s) a += mix[s * S + t] * x[s][i];
        nx[t][i] = a + outw[t] * yv[i];
      }
    }
#pragma unroll
    for (int t = 0; t < S; ++t) {
#pragma unroll
      for (int i = 0; i < V; ++i) x[t][i] = nx[t][i];
      if (!rows) store_v<float, V>(xr + (size_t)t * hidden, nx[t]);
    }
  }
  float u[V];
#pragma unroll
  for (int i = 0; i < V; ++i) {
    float a = 0.f;
#pragma unroll
    for (int s = 0; s < S; ++s) a += inw[s] * x[s][i];
    u[i] = norm_kind == 1 ? tanhf(alpha * a) * wv[i] + bv[i] : a;
  }
  store_v<T, V>(normed + (size_t)out_row * hidden + c, u);
}

// Dynamic Tanh on a single stream of the working type, with the residual sum in front of it as the
// RMSNorm kernel has it: with delta, x <- round(x + delta) first (written back unless rows is given).
template <typename T>
__global__ void dyt_kernel(T* __restrict__ x, const T* __restrict__ delta, const float* __restrict__ alpha_p,
                           const float* __restrict__ w, const float* __restrict__ b, T* __restrict__ y,
                           const int* __restrict__ rows, int hidden) {
  const float alpha = alpha_p[0];
  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(delta);
  SB_BEHIND_WAIT(rows);
  const int out_row = blockIdx.x;
  const int in_row = rows ? rows[out_row] : out_row;
  T* xr = x + (size_t)in_row * hidden;
  const T* dr = delta ? delta + (size_t)in_row * hidden : nullptr;
  T* yr = y + (size_t)out_row * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = to_f<T>(xr[c]);
    if (dr) {
      v = rnd<T>(v + to_f<T>(dr[c]));
      if (!rows) xr[c] = from_f<T>(v);
    }
    yr[c] = from_f<T>(tanhf(alpha * v) * w[c] + b[c]);
  }
}

template <typename T>
__global__ void add_bias_kernel(T* __restrict__ y, const float* __restrict__ bias, int width, size_t total) {
  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(y);
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) y[i] = from_f<T>(to_f<T>(y[i]) + bias[i % width]);
}

template <typename T, int V>
static int launch_step_v(int S, float* streams, const void* y, const float* y_bias, const float* mix_prev,
                         const float* out_prev, const float* in_next, int norm_kind, const float* alpha,
                         const float* w, const float* b, void* normed, const int* rows, int n_rows, int hidden,
                         cudaStream_t s) {
  const int threads = 128;
  const dim3 grid(n_rows, (hidden + threads * V - 1) / (threads * V));
#define GO(N) case N: return launch_dependent(hyper_step_kernel<T, N, V>, grid, dim3(threads), 0, s, streams, \
    (const T*)y, y_bias, mix_prev, out_prev, in_next, norm_kind, alpha, w, b, (T*)normed, rows, hidden)
  switch (S) {
    GO(1); GO(2); GO(3); GO(4); GO(5); GO(6); GO(7); GO(8);
  }
#undef GO
  return -2;
}

template <typename T>
static int launch_step(int S, float* streams, const void* y, const float* y_bias, const float* mix_prev,
                       const float* out_prev, const float* in_next, int norm_kind, const float* alpha,
                       const float* w, const float* b, void* normed, const int* rows, int n_rows, int hidden,
                       cudaStream_t s) {
  const uintptr_t all = (uintptr_t)streams | (uintptr_t)y | (uintptr_t)y_bias | (uintptr_t)w | (uintptr_t)b | (uintptr_t)normed;
  if (hidden % 4 == 0 && (all & 15) == 0)
    return launch_step_v<T, 4>(S, streams, y, y_bias, mix_prev, out_prev, in_next, norm_kind, alpha, w, b, normed, rows, n_rows, hidden, s);
  return launch_step_v<T, 1>(S, streams, y, y_bias, mix_prev, out_prev, in_next, norm_kind, alpha, w, b, normed, rows, n_rows, hidden, s);
}

extern "C" {

int sb_max_streams() { return SB_MAX_STREAMS; }

// out: float [n_tokens, streams, hidden], every stream the token's embedding.  serial != 0: an
// ordinary launch (the step's fence, see sb_embedding).
int sb_embed_streams(int dtype, const int* tokens, const void* table, float* out, int n_tokens, int hidden,
                     int vocab, int streams, int* status, int serial, cudaStream_t s) {
  if (n_tokens == 0) return 0;
  if (streams < 1) return -2;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (serial) {
    if (dtype == 0)
      embed_streams_kernel<float><<<n_tokens, threads, 0, s>>>(tokens, (const float*)table, out, hidden, vocab, streams, status);
    else
      embed_streams_kernel<bf16><<<n_tokens, threads, 0, s>>>(tokens, (const bf16*)table, out, hidden, vocab, streams, status);
    return SB_LAUNCH_RESULT();
  }
  if (dtype == 0)
    return launch_dependent(embed_streams_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, tokens, (const float*)table, out, hidden, vocab, streams, status);
  return launch_dependent(embed_streams_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, s, tokens, (const bf16*)table, out, hidden, vocab, streams, status);
}

// streams: float [*, S, hidden].  y (null: no pending update) [*, hidden] of the working type, y_bias
// null or float [hidden]; mix_prev [S, S] ([from][to]), out_prev [S]; in_next [S] or null (plain sum).
// normed: [n_rows, hidden] of the working type.  rows null: every row, updated in place; else only
// those rows and nothing is written back.
int sb_hyper_step(int dtype, int n_streams, float* streams, const void* y, const float* y_bias,
                  const float* mix_prev, const float* out_prev, const float* in_next, int norm_kind,
                  const float* alpha, const float* w, const float* b, void* normed, const int* rows,
                  int n_rows, int hidden, cudaStream_t s) {
  if (n_rows == 0) return 0;
  if (n_streams < 1 || n_streams > SB_MAX_STREAMS) return -2;
  if (dtype == 0)
    return launch_step<float>(n_streams, streams, y, y_bias, mix_prev, out_prev, in_next, norm_kind, alpha, w, b, normed, rows, n_rows, hidden, s);
  return launch_step<bf16>(n_streams, streams, y, y_bias, mix_prev, out_prev, in_next, norm_kind, alpha, w, b, normed, rows, n_rows, hidden, s);
}

int sb_add_bias(int dtype, void* y, const float* bias, int n_rows, int width, cudaStream_t s) {
  const size_t total = (size_t)n_rows * width;
  if (total == 0) return 0;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == 0)
    return launch_dependent(add_bias_kernel<float>, dim3((int)blocks), dim3(256), 0, s, (float*)y, bias, width, total);
  return launch_dependent(add_bias_kernel<bf16>, dim3((int)blocks), dim3(256), 0, s, (bf16*)y, bias, width, total);
}

int sb_dyt(int dtype, void* x, const void* delta, const float* alpha, const float* w, const float* b, void* y,
           const int* rows, int n_rows, int hidden, cudaStream_t s) {
  if (n_rows == 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (dtype == 0)
    return launch_dependent(dyt_kernel<float>, dim3(n_rows), dim3(threads), 0, s, (float*)x, (const float*)delta, alpha, w, b, (float*)y, rows, hidden);
  return launch_dependent(dyt_kernel<bf16>, dim3(n_rows), dim3(threads), 0, s, (bf16*)x, (const bf16*)delta, alpha, w, b, (bf16*)y, rows, hidden);
}

}  // extern "C"
