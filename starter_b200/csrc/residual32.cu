// A residual stream kept in 32-bit floats whatever the working type, for layers with a norm on both
// sides of each sublayer:
//
//     x <- x + post(sublayer(pre(x)))          pre, post: RMS norms with gains of their own
//
// The sum that closes one sublayer and the norm that opens the next touch the same row, so they are
// ONE kernel (as the residual sum and the norm after it are one kernel in the models whose residual
// has the working type): residual_norm takes the sublayer's output y (working type, with an optional
// float bias that was left for it to add), norms it with the post gain, adds it onto the float row
// in place, and norms the new row with the next sublayer's gain into the working type.  With `rows`
// it does the same for selected rows without writing back: that closes the model.
//
// Norm: y / sqrt(mean(y^2) + eps) * gain, everything in float; the gain arrives as a float vector
// (a gain stored around zero has had its one added when the weights were loaded).
//
// Also here: the embedding gather into such a stream (times a constant), and the bias + activation
// of a dense feed-forward whose projections have biases.
#include "common.cuh"

template <typename T>
__global__ void embed32_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                               float* __restrict__ out, int hidden, int vocab, float scale, int* status) {
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
  SB_BEHIND_WAIT(tokens);
  const int row = blockIdx.x;
  int tok = tokens[row];
  const bool bad = tok < 0 || tok >= vocab;
  if (bad) {
    if (threadIdx.x == 0 && status) atomicOr(status, 1);
    tok = 0;
  }
  const T* src = table + (size_t)tok * hidden;
  float* dst = out + (size_t)row * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = bad ? 0.f : to_f<T>(src[c]) * scale;
}

// One block per row; the row lives in shared memory (hidden floats) between the passes.
template <typename T>
__global__ void residual_norm_kernel(float* __restrict__ x, const T* __restrict__ y,
                                     const float* __restrict__ y_bias, const float* __restrict__ post_gain,
                                     const float* __restrict__ next_gain, T* __restrict__ out,
                                     const int* __restrict__ rows, int hidden, float eps_post, float eps) {
  extern __shared__ float row[];
  __shared__ float scratch[33];
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
  SB_BEHIND_WAIT(y);
  SB_BEHIND_WAIT(rows);
  SB_BEHIND_WAIT(x);
  const int out_row = blockIdx.x;
  const int in_row = rows ? rows[out_row] : out_row;
  float* xr = x + (size_t)in_row * hidden;
  float sq = 0.f;
  if (y) {
    const T* yr = y + (size_t)in_row * hidden;
    float ysq = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      float v = to_f<T>(yr[c]);
      if (y_bias) v += y_bias[c];
      row[c] = v;
      ysq += v * v;
    }
    ysq = block_sum(ysq, scratch);
    const float inv = post_gain ? 1.f / sqrtf(ysq / (float)hidden + eps_post) : 1.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      const float d = post_gain ? row[c] * inv * post_gain[c] : row[c];
      const float v = xr[c] + d;
      if (!rows) xr[c] = v;
      row[c] = v;
      sq += v * v;
    }
  } else {
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      const float v = xr[c];
      row[c] = v;
      sq += v * v;
    }
  }
  if (!out) return;
  sq = block_sum(sq, scratch);
  const float inv = 1.f / sqrtf(sq / (float)hidden + eps);
  T* o = out + (size_t)out_row * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) o[c] = from_f<T>(row[c] * inv * next_gain[c]);
}

// y[r, c] = act(x[r, c] + bias[c]); act 0: none, 1: relu, squared; 2: tanh; 3: exp(-exp(.)), the decay
// of a recurrence from its logarithm's logarithm.
template <typename T>
__global__ void bias_act_kernel(const T* __restrict__ x, const float* __restrict__ bias, T* __restrict__ y,
                                int width, size_t total, int act) {
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
  SB_BEHIND_WAIT(x);
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    float v = to_f<T>(x[i]);
    if (bias) v += bias[i % width];
    if (act == 1) {
      v = fmaxf(v, 0.f);
      v = v * v;
    } else if (act == 2) {
      v = tanhf(v);
    } else if (act == 3) {
      v = expf(-expf(v));
    }
    y[i] = from_f<T>(v);
  }
}

extern "C" {

// out: float [n_tokens, hidden] = table[token] * scale.  serial != 0: an ordinary launch (the step's
// fence: everything earlier steps wrote is complete before any kernel of this step starts).
int sb_embed32(int dtype, const int* tokens, const void* table, float* out, int n_tokens, int hidden,
               int vocab, float scale, int* status, int serial, cudaStream_t s) {
  if (n_tokens == 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (serial) {
    if (dtype == 0)
      embed32_kernel<float><<<n_tokens, threads, 0, s>>>(tokens, (const float*)table, out, hidden, vocab, scale, status);
    else
      embed32_kernel<bf16><<<n_tokens, threads, 0, s>>>(tokens, (const bf16*)table, out, hidden, vocab, scale, status);
    return SB_LAUNCH_RESULT();
  }
  if (dtype == 0)
    return launch_dependent(embed32_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, tokens, (const float*)table, out, hidden, vocab, scale, status);
  return launch_dependent(embed32_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, s, tokens, (const bf16*)table, out, hidden, vocab, scale, status);
}

// x: float [*, hidden].  y (null: nothing to add) [*, hidden] of the working type; y_bias null or float
// [hidden]; post_gain float [hidden] or null (y is added as it is).  next_gain / out: the norm of the
// new row into the working type (out null: only the sum).  rows null: every row, x updated in place.
// eps_post belongs to the norm of y, eps to the norm of the new row.
int sb_residual_norm(int dtype, float* x, const void* y, const float* y_bias, const float* post_gain,
                     const float* next_gain, void* out, const int* rows, int n_rows, int hidden, float eps_post,
                     float eps, cudaStream_t s) {
  if (n_rows == 0) return 0;
  if (out && !next_gain) return -2;
  const size_t smem = (size_t)hidden * sizeof(float);
  if (smem > 200 * 1024) return -2;
  const int threads = hidden >= 2048 ? 512 : hidden >= 512 ? 256 : 128;
  if (dtype == 0) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(residual_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_dependent(residual_norm_kernel<float>, dim3(n_rows), dim3(threads), smem, s, x, (const float*)y,
                            y_bias, post_gain, next_gain, (float*)out, rows, hidden, eps_post, eps);
  }
  if (smem > 48 * 1024) cudaFuncSetAttribute(residual_norm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return launch_dependent(residual_norm_kernel<bf16>, dim3(n_rows), dim3(threads), smem, s, x, (const bf16*)y,
                          y_bias, post_gain, next_gain, (bf16*)out, rows, hidden, eps_post, eps);
}

int sb_bias_act(int dtype, const void* x, const float* bias, void* y, int n_rows, int width, int act,
                cudaStream_t s) {
  const size_t total = (size_t)n_rows * width;
  if (total == 0) return 0;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == 0)
    return launch_dependent(bias_act_kernel<float>, dim3((int)blocks), dim3(256), 0, s, (const float*)x, bias, (float*)y, width, total, act);
  return launch_dependent(bias_act_kernel<bf16>, dim3((int)blocks), dim3(256), 0, s, (const bf16*)x, bias, (bf16*)y, width, total, act);
}

}  // extern "C"
