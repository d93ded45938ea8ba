// A linear recurrence with a matrix state per head and a decay that depends on the token (the time
// mixing of the RWKV family), over packed sequences, with the state kept per cache slot.
//
// Per head, with r, k, v, w of `dim` entries each for token t and a bonus vector u:
//
//     o_t[j] = sum_i r_t[i] * (S[i][j] + u[i] * k_t[i] * v_t[j])          S before this token
//     S[i][j] <- w_t[i] * S[i][j] + k_t[i] * v_t[j]
//     w_t[i]  = exp(-exp(x_t[i] + w0[i]))                                  x: the decay projection;
//                                                                          formed before this kernel
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
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
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

// Thread (j, p) holds S[i][j] for the KPT consecutive i from p * KPT.  P is a power of two (at most 32),
// the P threads of a j are neighbouring lanes and sum their parts of o[j] by shuffles.  VEC: dim is a
// multiple of 4 and a thread's r, k, w come from shared memory four at a time.
template <typename T, int KPT, bool VEC, int PF, int DC, int CH>
__global__ void __launch_bounds__(KPT > 32 ? 1024 : 512)
wkv_scan_kernel(const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v,
                const float* __restrict__ decay, const float* __restrict__ u,
                const T* __restrict__ g, const float* __restrict__ gain, float* __restrict__ state,
                size_t state_stride, int state_offset, const T* __restrict__ h, int width, T* __restrict__ out,
                const int* __restrict__ seq_slot, const int* __restrict__ seq_q_start,
                const int* __restrict__ seq_q_len, int heads, int D_arg, int P_arg, float eps,
                float* __restrict__ o32) {
  extern __shared__ __align__(16) float smem[];
  // DC != 0: the head size is known when the kernel is compiled and all index arithmetic folds away
  const int D = DC ? DC : D_arg, P = DC ? DC / KPT : P_arg;
  // gridDim.z blocks share a head: each owns D / gridDim.z of the state's columns j, and leaves its part
  // of o unnormed in o32 (float [tokens, heads * D]) for wkv_finish_kernel
  const int JW = D / (int)gridDim.z, j_base = blockIdx.z * JW;
  const int tid = threadIdx.x, nt = blockDim.x;
  const int seq = blockIdx.x, head = blockIdx.y;
  const int j = j_base + tid / P, p = tid % P;
  const bool live = tid / P < JW;
  const int hd = heads * D;
  const int i0 = p * KPT;
  // [2][4][CHUNK][D] inputs (r, k, w, v) and [CHUNK][D] outputs
  float* in_buf = smem;
  float* o_buf = smem + 2 * 4 * CH * D;
  float uu[KPT];
#pragma unroll
  for (int m = 0; m < KPT; ++m) uu[m] = (live && i0 + m < D) ? u[head * D + i0 + m] : 0.f;
  // which elements of a chunk this thread brings in: element e = tid + n * nt of [token][r | k | x | v][D]
  const int row4 = 4 * D;
  const int e_tt0 = tid / row4, e_col0 = tid - e_tt0 * row4;
  const int e_dtt = nt / row4, e_dcol = nt - e_dtt * row4;
  // (launch_dependents comes at this kernel's end, not its start: it runs in several waves of large blocks,
  // and a successor that starts early would only sit on the SMs its later waves need)
  pdl_wait();
  SB_BEHIND_WAIT(r); SB_BEHIND_WAIT(k); SB_BEHIND_WAIT(v); SB_BEHIND_WAIT(decay); SB_BEHIND_WAIT(g);
  SB_BEHIND_WAIT(state); SB_BEHIND_WAIT(h);
  SB_BEHIND_WAIT(seq_slot); SB_BEHIND_WAIT(seq_q_start); SB_BEHIND_WAIT(seq_q_len);
  const int slot = seq_slot[seq], q_start = seq_q_start[seq], q_len = seq_q_len[seq];
  float* held = state + (size_t)slot * state_stride;
  float* S_mem = held + state_offset + ((size_t)head * D + (live ? j : 0)) * D;
  float S[KPT];
#pragma unroll
  for (int m = 0; m < KPT; ++m) S[m] = (live && i0 + m < D) ? S_mem[i0 + m] : 0.f;
  const int per_chunk = 4 * CH * D;
  const int n_chunks = (q_len + CH - 1) / CH;
  unsigned pre[PF];   // PF * blockDim.x covers a chunk's elements; raw bits, converted when they are filed

  // Loads are issued here and their values first touched in stash(), a chunk's worth of work later:
  // nothing in between waits for them.  With the head size compiled in, a thread brings in 16-byte pieces
  // (piece q of a token: the r, k, v rows, then the decay row); else single elements.
  constexpr int TPP = 16 / (int)sizeof(T);                     // elements of r, k, v in a piece
  constexpr int NP = DC ? 3 * DC / TPP + DC / 4 : 1;           // pieces a token
  constexpr int NTC = KPT == 4 ? 256 : 512;                    // threads of the two launches that compile DC in
  constexpr int PV = DC ? (CH * NP + NTC - 1) / NTC : 1;
  uint4 prev[PV];
  auto fetch = [&](int chunk) {
    if (DC) {
#pragma unroll
      for (int n = 0; n < PV; ++n) {
        const int q = tid + n * nt;
        const int tt = q / NP, piece = q - tt * NP;
        const int t = chunk * CH + tt;
        prev[n] = make_uint4(0u, 0u, 0u, 0u);
        if (tt < CH && t < q_len) {
          const size_t row = (size_t)(q_start + t) * hd + head * D;
          if (piece < 3 * D / TPP) {
            const int a = piece / (D / TPP), off = (piece - a * (D / TPP)) * TPP;
            const T* src = a == 0 ? r : a == 1 ? k : v;
            prev[n] = *reinterpret_cast<const uint4*>(src + row + off);
          } else {
            prev[n] = *reinterpret_cast<const uint4*>(decay + row + (piece - 3 * D / TPP) * 4);
          }
        }
      }
      return;
    }
    int tt = e_tt0, col = e_col0;
#pragma unroll
    for (int n = 0; n < PF; ++n) {
      pre[n] = 0u;
      const int t = chunk * CH + tt;
      if (tt < CH && t < q_len) {
        const int a = (col >= D) + (col >= 2 * D) + (col >= 3 * D);
        const size_t at = (size_t)(q_start + t) * hd + head * D + (col - a * D);
        if (a == 2) {
          pre[n] = __float_as_uint(decay[at]);
        } else {
          const T* src = a == 0 ? r : a == 1 ? k : v;
          if (sizeof(T) == 2) pre[n] = reinterpret_cast<const unsigned short*>(src)[at];
          else pre[n] = reinterpret_cast<const unsigned*>(src)[at];
        }
      }
      tt += e_dtt;
      col += e_dcol;
      if (col >= row4) { col -= row4; ++tt; }
    }
  };
  auto stash = [&](int buf) {
    float* dst = in_buf + (size_t)buf * per_chunk;
    if (DC) {
#pragma unroll
      for (int n = 0; n < PV; ++n) {
        const int q = tid + n * nt;
        const int tt = q / NP, piece = q - tt * NP;
        if (tt >= CH) continue;
        const unsigned raw[4] = {prev[n].x, prev[n].y, prev[n].z, prev[n].w};
        if (piece < 3 * D / TPP) {
          const int a = piece / (D / TPP), off = (piece - a * (D / TPP)) * TPP;
          // the smem order of the arrays is r, k, decay, v
          float* row = dst + ((a == 2 ? 3 : a) * CH + tt) * D + off;
          if (sizeof(T) == 2) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              row[2 * i] = __uint_as_float(raw[i] << 16);
              row[2 * i + 1] = __uint_as_float(raw[i] & 0xffff0000u);
            }
          } else {
            *reinterpret_cast<uint4*>(row) = prev[n];
          }
        } else {
          *reinterpret_cast<uint4*>(dst + (2 * CH + tt) * D + (piece - 3 * D / TPP) * 4) = prev[n];
        }
      }
      return;
    }
    int tt = e_tt0, col = e_col0;
#pragma unroll
    for (int n = 0; n < PF; ++n) {
      if (tt < CH) {
        const int a = (col >= D) + (col >= 2 * D) + (col >= 3 * D);
        const int d = col - a * D;
        dst[(a * CH + tt) * D + d] = sizeof(T) == 2 && a != 2 ? __uint_as_float(pre[n] << 16) : __uint_as_float(pre[n]);
      }
      tt += e_dtt;
      col += e_dcol;
      if (col >= row4) { col -= row4; ++tt; }
    }
  };

  fetch(0);
  stash(0);
  __syncthreads();
  for (int c = 0; c < n_chunks; ++c) {
    const int buf = c & 1;
    if (c + 1 < n_chunks) fetch(c + 1);
    const float* rs = in_buf + (size_t)buf * per_chunk;
    const float* ks = rs + CH * D;
    const float* ws = ks + CH * D;
    const float* vs = ws + CH * D;
    const int here = min(CH, q_len - c * CH);
#pragma unroll 2
    for (int tt = 0; tt < here; ++tt) {
      const float vj = live ? vs[tt * D + j] : 0.f;
      float acc = 0.f;
      if (VEC) {
#pragma unroll
        for (int m = 0; m < KPT; m += 4) {
          if (i0 + m < D) {
            const float4 r4 = *reinterpret_cast<const float4*>(rs + tt * D + i0 + m);
            const float4 k4 = *reinterpret_cast<const float4*>(ks + tt * D + i0 + m);
            const float4 w4 = *reinterpret_cast<const float4*>(ws + tt * D + i0 + m);
            const float rr[4] = {r4.x, r4.y, r4.z, r4.w}, kk[4] = {k4.x, k4.y, k4.z, k4.w};
            const float ww[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float kv = kk[q] * vj;
              acc += rr[q] * (S[m + q] + uu[m + q] * kv);
              S[m + q] = ww[q] * S[m + q] + kv;
            }
          }
        }
      } else {
#pragma unroll
        for (int m = 0; m < KPT; ++m) {
          const int i = i0 + m;
          if (i < D) {
            const float kv = ks[tt * D + i] * vj;
            acc += rs[tt * D + i] * (S[m] + uu[m] * kv);
            S[m] = ws[tt * D + i] * S[m] + kv;
          }
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
        if (o < P) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (live && p == 0) o_buf[tt * D + j] = acc;
    }
    __syncthreads();
    if (gridDim.z > 1) {
      for (int e = tid; e < here * JW; e += nt) {
        const int tt = e / JW, d = j_base + e - tt * JW;
        o32[(size_t)(q_start + c * CH + tt) * hd + head * D + d] = o_buf[tt * D + d];
      }
    }
    // the head norm, the gain and the gate for this chunk's tokens: a warp a token
    for (int tt = tid >> 5; tt < (gridDim.z > 1 ? 0 : here); tt += nt >> 5) {
      const int lane = tid & 31;
      float sq = 0.f;
      for (int d = lane; d < D; d += 32) sq += o_buf[tt * D + d] * o_buf[tt * D + d];
      sq = warp_sum(sq);
      const float inv = 1.f / sqrtf(sq / (float)D + eps);
      const size_t at = (size_t)(q_start + c * CH + tt) * hd + head * D;
      for (int d = lane; d < D; d += 32) {
        const float gv = to_f<T>(g[at + d]);
        out[at + d] = from_f<T>(o_buf[tt * D + d] * inv * gain[head * D + d] * (gv / (1.f + expf(-gv))));
      }
    }
    if (c + 1 < n_chunks) stash(buf ^ 1);
    __syncthreads();
  }
  pdl_trigger();
#pragma unroll
  for (int m = 0; m < KPT; ++m)
    if (live && i0 + m < D) S_mem[i0 + m] = S[m];
  if (head == 0 && blockIdx.z == 0) {
    // the sequence's last mixer input: what the next portion's first token is shifted with
    const T* last = h + (size_t)(q_start + q_len - 1) * width;
    for (int c = tid; c < width; c += nt) held[c] = to_f<T>(last[c]);
  }
}

// The head norm, the gain and the gate over o32 when several blocks shared a head: a warp a (token, head).
template <typename T>
__global__ void wkv_finish_kernel(const float* __restrict__ o32, const T* __restrict__ g, const float* __restrict__ gain,
                                  T* __restrict__ out, int n_tokens, int heads, int D, float eps) {
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
  SB_BEHIND_WAIT(o32);
  SB_BEHIND_WAIT(g);
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= (long long)n_tokens * heads) return;
  const int head = (int)(warp % heads);
  const size_t at = (size_t)warp * D;
  float sq = 0.f;
  for (int d = lane; d < D; d += 32) sq += o32[at + d] * o32[at + d];
  sq = warp_sum(sq);
  const float inv = 1.f / sqrtf(sq / (float)D + eps);
  for (int d = lane; d < D; d += 32) {
    const float gv = to_f<T>(g[at + d]);
    out[at + d] = from_f<T>(o32[at + d] * inv * gain[head * D + d] * (gv / (1.f + expf(-gv))));
  }
}

struct ScanArgs {
  const void *r, *k, *v;
  const float *decay, *u;
  const void* g;
  const float* gain;
  float* state;
  size_t state_stride;
  int state_offset;
  const void* h;
  int width;
  void* out;
  const int *seq_slot, *seq_q_start, *seq_q_len;
  int n_seqs, heads, D;
  float eps;
  float* o32;
  int n_tokens;
};

template <typename T, int KPT, bool VEC, int PF, int DC, int CH>
static int launch_scan_as(const ScanArgs& a, int P, int threads, int j_split, cudaStream_t s) {
  const size_t smem = (size_t)(2 * 4 + 1) * CH * a.D * sizeof(float);
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(wkv_scan_kernel<T, KPT, VEC, PF, DC, CH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  int rc = launch_dependent(wkv_scan_kernel<T, KPT, VEC, PF, DC, CH>, dim3(a.n_seqs, a.heads, j_split), dim3(threads), smem,
                            s, (const T*)a.r, (const T*)a.k, (const T*)a.v, a.decay, a.u, (const T*)a.g, a.gain,
                            a.state, a.state_stride, a.state_offset, (const T*)a.h, a.width, (T*)a.out, a.seq_slot,
                            a.seq_q_start, a.seq_q_len, a.heads, a.D, P, a.eps, a.o32);
  if (rc != 0 || j_split == 1) return rc;
  const long long warps = (long long)a.n_tokens * a.heads;
  return launch_dependent(wkv_finish_kernel<T>, dim3((unsigned)((warps * 32 + 255) / 256)), dim3(256), 0, s,
                          (const float*)a.o32, (const T*)a.g, a.gain, (T*)a.out, a.n_tokens, a.heads, a.D, a.eps);
}

// Heads of up to 64 channels: 8 state values a thread; up to 128: 32; up to 256: 64 at 1,024 threads, which
// the compiler keeps partly in local memory (correct, and slower than the sizes below it).  Heads of
// exactly 64 channels have a kernel of their own with the size compiled in; with o32 given and few
// (sequence, head) pairs for the SMs there are, four blocks share a head (each a quarter of the state's
// columns with 16 threads a column) and a second kernel norms.
template <typename T>
static int launch_scan(const ScanArgs& a, cudaStream_t s) {
  const int D = a.D;
  if (D == 64) {
    const int j_split = (a.o32 && a.n_seqs * a.heads <= 74) ? 4 : 1;
    if (j_split == 4) return launch_scan_as<T, 4, true, 8, 64, 32>(a, 16, 256, 4, s);
    return launch_scan_as<T, 8, true, 8, 64, 16>(a, 8, 512, 1, s);
  }
  const int kpt = D <= 64 ? 8 : D <= 128 ? 32 : 64;
  int P = 1;
  while (P * kpt < D) P *= 2;
  int threads = (D * P + 31) / 32 * 32;
  const int need = (4 * WKV_CHUNK * D + threads - 1) / threads;      // elements of a chunk a thread brings in
  if (P > 32 || threads > (kpt > 32 ? 1024 : 512) || need > WKV_PREFETCH) return -2;
  const bool vec = D % 4 == 0;
#define GO(K, V, F) return launch_scan_as<T, K, V, F, 0, WKV_CHUNK>(a, P, threads, 1, s)
  if (kpt == 8 && need <= 8) { if (vec) GO(8, true, 8); GO(8, false, 8); }
  if (kpt == 8) { if (vec) GO(8, true, 32); GO(8, false, 32); }
  if (need > 16) return -2;
  if (kpt == 32) { if (vec) GO(32, true, 16); GO(32, false, 16); }
  if (vec) GO(64, true, 16);
  GO(64, false, 16);
#undef GO
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

// r, k, v, g, out: [n_tokens, heads * dim] of the working type; decay: float, same shape, the factors
// w_t themselves; gain: float [heads * dim]; u: float [heads, dim].  The state of a slot: see the head of this file
// (state_offset = where S starts inside a slot's floats).  o32: null, or float [n_tokens, heads * dim] of
// scratch, with which a step of few sequences may spread a head over several blocks (two launches).
int sb_wkv_scan(int dtype, const void* r, const void* k, const void* v, const float* decay,
                const float* u, const void* g, const float* gain, float* state, long long state_stride,
                int state_offset, const void* h, int width, void* out, const int* seq_slot, const int* seq_q_start,
                const int* seq_q_len, int n_seqs, int heads, int dim, float eps, float* o32, int n_tokens,
                cudaStream_t s) {
  if (n_seqs == 0) return 0;
  if (dim < 1 || dim > 256 || heads < 1) return -2;
  ScanArgs a = {r, k, v, decay, u, g, gain, state, (size_t)state_stride, state_offset, h, width, out,
                seq_slot, seq_q_start, seq_q_len, n_seqs, heads, dim, eps, o32, n_tokens};
  return dtype == 0 ? launch_scan<float>(a, s) : launch_scan<bf16>(a, s);
}

}  // extern "C"
