// Differential attention on tensor cores (bfloat16): the kernel for steps in which a sequence brings
// many tokens, and further down the one for single tokens.
//
// A block takes 64 queries of one query head (four warps of 16 rows) and walks the sequence's cache
// pages once.  A page's key rows hold both maps, [k1 | k2] of `dim` each, so the two score tiles
// S1 = Q1 K1^T and S2 = Q2 K2^T come from the same shared-memory tile (different 16-column steps of
// it); each map has its own running maximum, sum and accumulator, and a page's values are read from
// shared memory once for both maps' P V products.  At the end the block forms
//     o = O1 / l1 - lambda * O2 / l2,   o / sqrt(mean(o^2) + eps) * out_scale * sigmoid(gate)
// per row (a row's columns lie in the four lanes of a quad) and writes bfloat16.
// Scores, weights, sums and both accumulators are float; products use mma.sync.m16n8k16 (bf16 in,
// float accumulate); tiles are staged with cp.async, two pages in flight, in the swizzled layout of the
// single-map prompt kernel.  Sizes: dim a multiple of 16 up to 128, v_dim a multiple of 16 up to 128.
#include "common.cuh"

#define DP_BQ 64
#define DP_THREADS 128

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Distributed shared memory: the address of `addr` (shared window) in block `rank` of the cluster, a load
// from there, and the two cluster barriers (one that publishes this block's writes, one that does not).
__device__ __forceinline__ uint32_t cluster_addr(uint32_t addr, uint32_t rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(addr), "r"(rank));
  return a;
}
__device__ __forceinline__ float cluster_load(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ void cluster_rendezvous() {
  asm volatile("barrier.cluster.arrive.relaxed;\n\tbarrier.cluster.wait;" ::: "memory");
}

// Byte offset of 16-byte column `chunk` of `row` in a [rows][D] bfloat16 tile with swizzled columns.
template <int D> __device__ __forceinline__ int tile_offset(int row, int chunk) {
  constexpr int C = D / 8;
  const int sw = C >= 8 ? (row & 7) : ((row / (8 / C)) % C);
  return row * D * 2 + ((chunk ^ sw) << 4);
}

struct DiffPrefillTail {
  float lambda, out_scale, eps;
};

template <int QK, int VD>
__global__ void __launch_bounds__(DP_THREADS)
diff_prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ gate, int gate_stride,
                    bf16* __restrict__ out, const bf16* __restrict__ k_store, const bf16* __restrict__ v_store,
                    const int* __restrict__ block_table, int table_stride, const int* __restrict__ seq_slot,
                    const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                    const int* __restrict__ seq_kv_len, const int* __restrict__ tile_seq,
                    const int* __restrict__ tile_first, int heads, int kv_heads, float scale_log2, int window,
                    DiffPrefillTail tail) {
  constexpr int CQ = QK / 8, CV = VD / 8;
  constexpr int K_BYTES = SB_PAGE_TOKENS * QK * 2, V_BYTES = SB_PAGE_TOKENS * VD * 2;
  constexpr int KSTEPS = QK / 32;  // 16-column steps of one map's Q.K^T (dim / 16)
  constexpr int NBLK = VD / 8;     // 8-wide column blocks of the output
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* q_tile = smem;                       // [64][QK]
  uint8_t* k_tiles = smem + DP_BQ * QK * 2;     // 2 x [64][QK]
  uint8_t* v_tiles = k_tiles + 2 * K_BYTES;     // 2 x [64][VD]

  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(q);
  SB_BEHIND_WAIT(gate);
  SB_BEHIND_WAIT(k_store);
  SB_BEHIND_WAIT(v_store);
  const int tile = blockIdx.x, head = blockIdx.y;
  const int seq = tile_seq[tile];
  const int q_first = tile_first[tile];
  const int q_len = seq_q_len[seq], kv_len = seq_kv_len[seq];
  const int rows_valid = min(DP_BQ, q_len - q_first);
  const int pos0 = kv_len - q_len + q_first;    // absolute position of the tile's first query
  const int kvh = head / (heads / kv_heads);
  const int* pages = block_table + (size_t)seq_slot[seq] * table_stride;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  const int hi = pos0 + rows_valid - 1;                                   // last key any row sees
  int lo = 0;
  if (window > 0 && pos0 - window + 1 > 0) lo = pos0 - window + 1;        // first key any row sees
  const int page_lo = lo / SB_PAGE_TOKENS, page_hi = hi / SB_PAGE_TOKENS;
  const int n_tiles = page_hi - page_lo + 1;

  // ---- stage the queries (rows past the end repeat the last valid row; they are never written)
  const size_t q_stride = (size_t)heads * QK;
  {
    const bf16* src = q + ((size_t)seq_q_start[seq] + q_first) * q_stride + (size_t)head * QK;
    for (int idx = tid; idx < DP_BQ * CQ; idx += DP_THREADS) {
      const int r = idx / CQ, c = idx % CQ;
      const int rr = min(r, rows_valid - 1);
      cp_async16(q_tile + tile_offset<QK>(r, c), src + (size_t)rr * q_stride + c * 8);
    }
  }
  auto load_kv = [&](int t, int buf) {
    const int page = pages[page_lo + t];
    const bf16* ks = k_store + page_row(page, kvh, 0, kv_heads, QK);
    const bf16* vs = v_store + page_row(page, kvh, 0, kv_heads, VD);
    for (int idx = tid; idx < SB_PAGE_TOKENS * CQ; idx += DP_THREADS)
      cp_async16(k_tiles + buf * K_BYTES + tile_offset<QK>(idx / CQ, idx % CQ), ks + (size_t)idx * 8);
    for (int idx = tid; idx < SB_PAGE_TOKENS * CV; idx += DP_THREADS)
      cp_async16(v_tiles + buf * V_BYTES + tile_offset<VD>(idx / CV, idx % CV), vs + (size_t)idx * 8);
  };
  load_kv(0, 0);
  cp_commit();
  if (n_tiles > 1) load_kv(1, 1);
  cp_commit();
  cp_wait<1>();
  __syncthreads();

  float o[2][NBLK][4];
#pragma unroll
  for (int mp = 0; mp < 2; ++mp)
#pragma unroll
    for (int n = 0; n < NBLK; ++n) o[mp][n][0] = o[mp][n][1] = o[mp][n][2] = o[mp][n][3] = 0.f;
  float m_run[2][2] = {{-INFINITY, -INFINITY}, {-INFINITY, -INFINITY}}, l_run[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
  const int row_a = warp * 16 + (lane >> 2);     // this thread's rows: row_a and row_a + 8
  const int pos_a = pos0 + row_a, pos_b = pos_a + 8;
  const int q_row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;   // the row this lane addresses for ldmatrix

  for (int t = 0; t < n_tiles; ++t) {
    const int buf = t & 1;
    const uint8_t* kt = k_tiles + buf * K_BYTES;
    const uint8_t* vt = v_tiles + buf * V_BYTES;
    const int j0 = (page_lo + t) * SB_PAGE_TOKENS;
    const bool edge = j0 + SB_PAGE_TOKENS - 1 > pos0 || (window > 0 && j0 <= pos0 + DP_BQ - window);
    uint32_t pf[2][4][4];   // both maps' P as A fragments: 4 k-steps of 16 keys

#pragma unroll
    for (int mp = 0; mp < 2; ++mp) {
      // S = Q_m K_m^T for 64 keys: 8 blocks of 8 keys
      float s[8][4];
#pragma unroll
      for (int nb = 0; nb < 8; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        const int step = mp * KSTEPS + kk;       // which 16 columns of the [k1 | k2] row
        uint32_t qf[4];
        ldmatrix_x4(smem_u32(q_tile + tile_offset<QK>(q_row, 2 * step + (lane >> 4))), qf[0], qf[1], qf[2], qf[3]);
#pragma unroll
        for (int nb = 0; nb < 8; nb += 2) {
          uint32_t b0, b1, b2, b3;
          const int key = nb * 8 + (lane & 7) + (lane >> 4) * 8;
          ldmatrix_x4(smem_u32(kt + tile_offset<QK>(key, 2 * step + ((lane >> 3) & 1))), b0, b1, b2, b3);
          mma_bf16(s[nb], qf, b0, b1);
          mma_bf16(s[nb + 1], qf, b2, b3);
        }
      }
      // scale, mask, online softmax of this map
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = s[nb][e] * scale_log2;
          if (edge) {
            const int j = j0 + nb * 8 + (lane & 3) * 2 + (e & 1);
            const int p = (e & 2) ? pos_b : pos_a;
            if (j > p || (window > 0 && j <= p - window)) v = -INFINITY;
          }
          s[nb][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      }
      float alpha[2], m_use[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m_run[mp][h], mx[h]);
        m_use[h] = m_new == -INFINITY ? 0.f : m_new;
        alpha[h] = exp2f(m_run[mp][h] - m_use[h]);
        m_run[mp][h] = m_new;
      }
      float rs[2] = {0.f, 0.f};
#pragma unroll
      for (int nb = 0; nb < 8; ++nb) {
        const float p0 = exp2f(s[nb][0] - m_use[0]), p1 = exp2f(s[nb][1] - m_use[0]);
        const float p2 = exp2f(s[nb][2] - m_use[1]), p3 = exp2f(s[nb][3] - m_use[1]);
        rs[0] += p0 + p1;
        rs[1] += p2 + p3;
        pf[mp][nb >> 1][(nb & 1) * 2] = pack_bf16(p0, p1);
        pf[mp][nb >> 1][(nb & 1) * 2 + 1] = pack_bf16(p2, p3);
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) l_run[mp][h] = l_run[mp][h] * alpha[h] + rs[h];
#pragma unroll
      for (int n = 0; n < NBLK; ++n) {
        o[mp][n][0] *= alpha[0]; o[mp][n][1] *= alpha[0];
        o[mp][n][2] *= alpha[1]; o[mp][n][3] *= alpha[1];
      }
    }

    // O_m += P_m V: a value fragment is read once and feeds both maps
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
      for (int n = 0; n < NBLK; n += 2) {
        uint32_t b0, b1, b2, b3;
        const int key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        ldmatrix_x4_trans(smem_u32(vt + tile_offset<VD>(key, n + (lane >> 4))), b0, b1, b2, b3);
        mma_bf16(o[0][n], pf[0][kk], b0, b1);
        mma_bf16(o[0][n + 1], pf[0][kk], b2, b3);
        mma_bf16(o[1][n], pf[1][kk], b0, b1);
        mma_bf16(o[1][n + 1], pf[1][kk], b2, b3);
      }
    }

    // this buffer is free: fetch the page after next, then make sure the next one has landed
    __syncthreads();
    if (t + 2 < n_tiles) load_kv(t + 2, buf);
    cp_commit();
    cp_wait<1>();
    __syncthreads();
  }
  cp_wait<0>();

  // ---- finish: both maps' row sums over the quad, the difference, its unit norm, the gate
  float inv[2][2];
#pragma unroll
  for (int mp = 0; mp < 2; ++mp)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float l = l_run[mp][h];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      inv[mp][h] = 1.f / l;
    }
  float ss[2] = {0.f, 0.f};
#pragma unroll
  for (int n = 0; n < NBLK; ++n) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int h = e >> 1;
      const float d = o[0][n][e] * inv[0][h] - tail.lambda * (o[1][n][e] * inv[1][h]);
      o[0][n][e] = d;
      ss[h] += d * d;
    }
  }
  float norm[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    ss[h] += __shfl_xor_sync(0xffffffffu, ss[h], 1);
    ss[h] += __shfl_xor_sync(0xffffffffu, ss[h], 2);
    norm[h] = rsqrtf(ss[h] / (float)VD + tail.eps) * tail.out_scale;
  }
  const size_t o_stride = (size_t)heads * VD;
  const size_t first_row = (size_t)seq_q_start[seq] + q_first;
  bf16* dst = out + first_row * o_stride + (size_t)head * VD;
  const bf16* gsrc = gate ? gate + first_row * gate_stride + (size_t)head * VD : nullptr;
#pragma unroll
  for (int n = 0; n < NBLK; ++n) {
    const int col = n * 8 + (lane & 3) * 2;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = row_a + 8 * h;
      if (row < rows_valid) {
        float a = o[0][n][2 * h] * norm[h], b = o[0][n][2 * h + 1] * norm[h];
        if (gsrc) {
          const __nv_bfloat162 g = *reinterpret_cast<const __nv_bfloat162*>(gsrc + (size_t)row * gate_stride + col);
          a *= 1.f / (1.f + __expf(-__bfloat162float(g.x)));
          b *= 1.f / (1.f + __expf(-__bfloat162float(g.y)));
        }
        *reinterpret_cast<uint32_t*>(dst + (size_t)row * o_stride + col) = pack_bf16(a, b);
      }
    }
  }
}

// ------------------------------------------------------------------------------------ single tokens
//
// One new token per sequence: the 16 MMA rows are the query heads that share a key/value head (more
// than 16: chunks of 16), so a page's keys and values are read once for all of them and for both maps.
// A block takes one (row, key/value head, part of the keys); its four warps share each page, 16 keys
// a warp, through a three-stage cp.async ring; every warp keeps its own running maximum, sum and
// accumulators per map, the warps' results meet in shared memory, and the block leaves its part as
// (maximum, sum, accumulator) per head and map in scratch memory.  diff_decode_merge joins the parts
// and finishes the head (difference, unit norm, gate).
//
// CLUSTER: the parts of a (row, key/value head) are the blocks of one thread-block cluster (n_splits
// <= 8).  Each leaves its part in its own shared memory; after a cluster barrier block s joins and
// finishes the heads s, s + n_splits, ... (a warp a head, reading every block's part through
// distributed shared memory), so there is neither scratch memory nor a second launch.
#define DD_STAGES 3
#define DD_CLUSTER_MAX 8

// own: this block's part, [16 heads][2 maps][VD + 2] floats (maximum, sum, accumulator) in shared memory
// at the same address in every block of the cluster.
template <int VD>
__device__ __forceinline__ void diff_decode_cluster_finish(const float* own, int split, int n_splits, int n_heads,
                                                           int row, int heads, int head0, const bf16* gate,
                                                           int gate_stride, bf16* out, const DiffPrefillTail& tail) {
  constexpr int PER = VD + 2, CPL = VD / 32;      // CPL columns a lane: lane, lane + 32, ...
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the gate's values are asked for ahead of the barrier and of the remote loads (of a head's, a pass ahead)
  float g[CPL];
  auto ask_gate = [&](int r) {
#pragma unroll
    for (int i = 0; i < CPL; ++i)
      g[i] = gate && r < n_heads ? __bfloat162float(gate[(size_t)row * gate_stride + (size_t)(head0 + r) * VD + lane + 32 * i]) : 0.f;
  };
  ask_gate(split + n_splits * warp);
  cluster_sync();                                  // every block's part is written and visible
  const uint32_t base = smem_u32(own);
  for (int r = split + n_splits * warp; r < n_heads; r += n_splits * (DP_THREADS / 32)) {
    float gv[CPL];
#pragma unroll
    for (int i = 0; i < CPL; ++i) gv[i] = g[i];
    ask_gate(r + n_splits * (DP_THREADS / 32));
    // every part's values first (the remote loads are in flight together), then the arithmetic; an empty
    // part holds (-inf, 0, zeros) and gets the weight 0
    float m[2][DD_CLUSTER_MAX], l[2][DD_CLUSTER_MAX], av[2][DD_CLUSTER_MAX][CPL];
#pragma unroll
    for (int sp = 0; sp < DD_CLUSTER_MAX; ++sp) {
      if (sp < n_splits) {
#pragma unroll
        for (int mp = 0; mp < 2; ++mp) {
          const uint32_t at = cluster_addr(base + (uint32_t)((r * 2 + mp) * PER) * 4u, sp);
          m[mp][sp] = cluster_load(at);
          l[mp][sp] = cluster_load(at + 4u);
#pragma unroll
          for (int i = 0; i < CPL; ++i) av[mp][sp][i] = cluster_load(at + (uint32_t)(2 + lane + 32 * i) * 4u);
        }
      }
    }
    float big[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int sp = 0; sp < DD_CLUSTER_MAX; ++sp)
      if (sp < n_splits) { big[0] = fmaxf(big[0], m[0][sp]); big[1] = fmaxf(big[1], m[1][sp]); }
    float den[2] = {0.f, 0.f}, a[2][CPL];
#pragma unroll
    for (int i = 0; i < CPL; ++i) a[0][i] = a[1][i] = 0.f;
#pragma unroll
    for (int sp = 0; sp < DD_CLUSTER_MAX; ++sp) {
      if (sp < n_splits) {
#pragma unroll
        for (int mp = 0; mp < 2; ++mp) {
          const float w = m[mp][sp] == -INFINITY ? 0.f : exp2f(m[mp][sp] - big[mp]);
          den[mp] += l[mp][sp] * w;
#pragma unroll
          for (int i = 0; i < CPL; ++i) a[mp][i] += av[mp][sp][i] * w;
        }
      }
    }
    float d[CPL], ss = 0.f;
#pragma unroll
    for (int i = 0; i < CPL; ++i) {
      d[i] = a[0][i] / den[0] - tail.lambda * (a[1][i] / den[1]);
      ss += d[i] * d[i];
    }
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, sh);
    const float norm = rsqrtf(ss / (float)VD + tail.eps) * tail.out_scale;
    const int head = head0 + r;
#pragma unroll
    for (int i = 0; i < CPL; ++i) {
      const int c = lane + 32 * i;
      float v = d[i] * norm;
      if (gate) v *= 1.f / (1.f + __expf(-gv[i]));
      out[((size_t)row * heads + head) * VD + c] = __float2bfloat16_rn(v);
    }
  }
  cluster_rendezvous();                            // nobody leaves while its shared memory is still read
}

template <int QK, int VD, bool CLUSTER>
__global__ void __launch_bounds__(DP_THREADS)
diff_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_store, const bf16* __restrict__ v_store,
                   const int* __restrict__ block_table, int table_stride, const int* __restrict__ row_slot,
                   const int* __restrict__ row_kv_len, int heads, int kv_heads, float scale_log2, int window,
                   int n_splits, float* __restrict__ part, int early, const bf16* __restrict__ gate,
                   int gate_stride, bf16* __restrict__ out, DiffPrefillTail tail) {
  constexpr int CQ = QK / 8, CV = VD / 8;
  constexpr int K_BYTES = SB_PAGE_TOKENS * QK * 2, V_BYTES = SB_PAGE_TOKENS * VD * 2;
  constexpr int KSTEPS = QK / 32, NBLK = VD / 8, PER = VD + 2;
  // a warp's rows in the meeting area lie VD + 8 floats apart: a quad writes 8 consecutive floats and the rows
  // of a half warp are 8 banks apart, so its 8-byte stores meet no bank twice
  constexpr int MPER = VD + 8;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* q_tile = smem;                            // [16][QK]
  uint8_t* k_tiles = smem + 16 * QK * 2;             // DD_STAGES x [64][QK]
  uint8_t* v_tiles = k_tiles + DD_STAGES * K_BYTES;  // DD_STAGES x [64][VD]
  float* meet = reinterpret_cast<float*>(k_tiles);   // after the walk: [4 warps][2 maps][16 rows][MPER]
  float* own = meet + 4 * 2 * 16 * MPER;             // CLUSTER: this block's part, [16 rows][2 maps][PER]
  // -DDD_TIMELINE (a build of its own, for measuring; the library never makes it): thread 0 of every block
  // leaves the global timer at the ends of its phases, and its SM, in `part`.
#ifdef DD_TIMELINE
  unsigned long long tl[8];
#define TL(k) do { asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tl[k])); } while (0)
  TL(0);
#else
#define TL(k)
#endif

  pdl_trigger();
  // `early`: the caller vouches that the rows' lengths, the page table and every cached key and value
  // but the newest token's were complete before this step's first kernel started, and that nothing
  // else in this step writes them.  Then the first pages (all but a row's last one, which holds the
  // token this step has just filed) are asked for before the dependent-launch wait, while the kernels
  // before this one still run.
  if (!early) {
    pdl_wait();
    SB_BEHIND_WAIT(row_slot);
    SB_BEHIND_WAIT(row_kv_len);
  }
  const int group = heads / kv_heads, chunks = (group + 15) / 16;
  const int split = blockIdx.x, kvh = blockIdx.y / chunks, chunk = blockIdx.y % chunks, row = blockIdx.z;
  const int head0 = kvh * group + chunk * 16, n_heads = min(16, group - chunk * 16);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int pos = row_kv_len[row] - 1;
  int lo = 0;
  if (window > 0 && pos - window + 1 > 0) lo = pos - window + 1;
  const int page_lo = lo / SB_PAGE_TOKENS, page_hi = pos / SB_PAGE_TOKENS;
  const int per = (page_hi - page_lo + n_splits) / n_splits;
  const int p_begin = page_lo + split * per, p_end = min(page_hi + 1, p_begin + per);
  const int n_pages = p_end - p_begin;
  float* mine = part + (((size_t)row * heads + head0) * n_splits + split) * 2 * PER;   // + r * n_splits * 2 * PER per head
  if (n_pages <= 0) {      // more parts than pages: this part is empty
    if (early) pdl_wait();
    if (CLUSTER) {
      SB_BEHIND_WAIT(gate);
      for (int i = tid; i < 16 * 2 * PER; i += DP_THREADS) own[i] = i % PER == 0 ? -INFINITY : 0.f;
      diff_decode_cluster_finish<VD>(own, split, n_splits, n_heads, row, heads, head0, gate, gate_stride, out, tail);
      return;
    }
    for (int i = tid; i < n_heads * 2; i += DP_THREADS) {
      float* dst = mine + (size_t)(i >> 1) * n_splits * 2 * PER + (i & 1) * PER;
      dst[0] = -INFINITY;
      dst[1] = 0.f;
    }
    return;
  }
  const int* pages = block_table + (size_t)row_slot[row] * table_stride;
  // A page's number is asked for a whole iteration before its copies are issued: the lookup's latency
  // (the table lies in L2 at best) would otherwise sit in front of every iteration's prefetch.
  int first_pages[DD_STAGES];
#pragma unroll
  for (int st = 0; st < DD_STAGES; ++st) first_pages[st] = st < n_pages ? pages[p_begin + st] : 0;
  int page_next = first_pages[DD_STAGES - 1];
  auto load_kv = [&](int page, int buf) {
    const bf16* ks = k_store + page_row(page, kvh, 0, kv_heads, QK);
    const bf16* vs = v_store + page_row(page, kvh, 0, kv_heads, VD);
    for (int idx = tid; idx < SB_PAGE_TOKENS * CQ; idx += DP_THREADS)
      cp_async16(k_tiles + buf * K_BYTES + tile_offset<QK>(idx / CQ, idx % CQ), ks + (size_t)idx * 8);
    for (int idx = tid; idx < SB_PAGE_TOKENS * CV; idx += DP_THREADS)
      cp_async16(v_tiles + buf * V_BYTES + tile_offset<VD>(idx / CV, idx % CV), vs + (size_t)idx * 8);
  };
  // before the wait: the pages of the first stages that earlier steps filled
  bool asked[DD_STAGES - 1];
#pragma unroll
  for (int s = 0; s < DD_STAGES - 1; ++s) {
    asked[s] = early && s < n_pages && p_begin + s < page_hi;
    if (asked[s]) load_kv(first_pages[s], s);
  }
  TL(1);
  if (early) pdl_wait();
  TL(2);
  SB_BEHIND_WAIT(q);
  SB_BEHIND_WAIT(k_store);
  SB_BEHIND_WAIT(v_store);
  {
    const bf16* src = q + (size_t)row * heads * QK;
    for (int idx = tid; idx < 16 * CQ; idx += DP_THREADS) {
      const int r = idx / CQ, c = idx % CQ;
      cp_async16(q_tile + tile_offset<QK>(r, c), src + (size_t)(head0 + min(r, n_heads - 1)) * QK + c * 8);
    }
  }
#pragma unroll
  for (int s = 0; s < DD_STAGES - 1; ++s)
    if (!asked[s] && s < n_pages) load_kv(first_pages[s], s);
  cp_commit();                       // one group: the queries and the first stages
  cp_wait<0>();
  TL(3);

  float o[2][NBLK][4];
#pragma unroll
  for (int mp = 0; mp < 2; ++mp)
#pragma unroll
    for (int n = 0; n < NBLK; ++n) o[mp][n][0] = o[mp][n][1] = o[mp][n][2] = o[mp][n][3] = 0.f;
  float m_run[2][2] = {{-INFINITY, -INFINITY}, {-INFINITY, -INFINITY}}, l_run[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
  const int q_row = (lane & 7) + ((lane >> 3) & 1) * 8;

  for (int t = 0; t < n_pages; ++t) {
    // the first DD_STAGES - 1 pages came in one group, awaited above; page t >= DD_STAGES - 1 is the group
    // committed DD_STAGES - 1 iterations ago, so all but the newest DD_STAGES - 2 groups must be done
    cp_wait<DD_STAGES - 2>();
    __syncthreads();                 // page t has landed for everyone, and everyone is done with page t - 1
    if (t + DD_STAGES - 1 < n_pages) load_kv(page_next, (t + DD_STAGES - 1) % DD_STAGES);
    cp_commit();
    if (t + DD_STAGES < n_pages) page_next = pages[p_begin + t + DD_STAGES];
    const int buf = t % DD_STAGES;
    const uint8_t* kt = k_tiles + buf * K_BYTES;
    const uint8_t* vt = v_tiles + buf * V_BYTES;
    const int j0 = (p_begin + t) * SB_PAGE_TOKENS + 16 * warp;      // this warp's 16 keys
    if (j0 > pos || (window > 0 && j0 + 15 <= pos - window)) continue;   // none of them is seen
    const bool edge = j0 + 15 > pos || (window > 0 && j0 <= pos - window);
    uint32_t pf[2][4];
#pragma unroll
    for (int mp = 0; mp < 2; ++mp) {
      float s[2][4];
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        const int step = mp * KSTEPS + kk;
        uint32_t qf[4], b0, b1, b2, b3;
        ldmatrix_x4(smem_u32(q_tile + tile_offset<QK>(q_row, 2 * step + (lane >> 4))), qf[0], qf[1], qf[2], qf[3]);
        const int key = 16 * warp + (lane & 7) + (lane >> 4) * 8;
        ldmatrix_x4(smem_u32(kt + tile_offset<QK>(key, 2 * step + ((lane >> 3) & 1))), b0, b1, b2, b3);
        mma_bf16(s[0], qf, b0, b1);
        mma_bf16(s[1], qf, b2, b3);
      }
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = s[nb][e] * scale_log2;
          if (edge) {
            const int j = j0 + nb * 8 + (lane & 3) * 2 + (e & 1);
            if (j > pos || (window > 0 && j <= pos - window)) v = -INFINITY;
          }
          s[nb][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      }
      float alpha[2], m_use[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m_run[mp][h], mx[h]);
        m_use[h] = m_new == -INFINITY ? 0.f : m_new;
        alpha[h] = exp2f(m_run[mp][h] - m_use[h]);
        m_run[mp][h] = m_new;
      }
      float rs[2] = {0.f, 0.f};
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
        const float p0 = exp2f(s[nb][0] - m_use[0]), p1 = exp2f(s[nb][1] - m_use[0]);
        const float p2 = exp2f(s[nb][2] - m_use[1]), p3 = exp2f(s[nb][3] - m_use[1]);
        rs[0] += p0 + p1;
        rs[1] += p2 + p3;
        pf[mp][nb * 2] = pack_bf16(p0, p1);
        pf[mp][nb * 2 + 1] = pack_bf16(p2, p3);
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) l_run[mp][h] = l_run[mp][h] * alpha[h] + rs[h];
#pragma unroll
      for (int n = 0; n < NBLK; ++n) {
        o[mp][n][0] *= alpha[0]; o[mp][n][1] *= alpha[0];
        o[mp][n][2] *= alpha[1]; o[mp][n][3] *= alpha[1];
      }
    }
#pragma unroll
    for (int n = 0; n < NBLK; n += 2) {
      uint32_t b0, b1, b2, b3;
      const int key = 16 * warp + (lane & 7) + ((lane >> 3) & 1) * 8;
      ldmatrix_x4_trans(smem_u32(vt + tile_offset<VD>(key, n + (lane >> 4))), b0, b1, b2, b3);
      mma_bf16(o[0][n], pf[0], b0, b1);
      mma_bf16(o[0][n + 1], pf[0], b2, b3);
      mma_bf16(o[1][n], pf[1], b0, b1);
      mma_bf16(o[1][n + 1], pf[1], b2, b3);
    }
  }
  cp_wait<0>();
  TL(4);
  __syncthreads();        // the ring is free: the warps' results meet in it

#pragma unroll
  for (int mp = 0; mp < 2; ++mp) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float l = l_run[mp][h];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      const int r = (lane >> 2) + 8 * h;
      float* dst = meet + ((warp * 2 + mp) * 16 + r) * MPER;
      if (r >= n_heads) continue;        // a row past the heads of this chunk: nobody reads it
      if ((lane & 3) == 0) { dst[0] = m_run[mp][h]; dst[1] = l; }
#pragma unroll
      for (int n = 0; n < NBLK; ++n) {
        const int col = n * 8 + (lane & 3) * 2;
        *reinterpret_cast<float2*>(dst + 2 + col) = make_float2(o[mp][n][2 * h], o[mp][n][2 * h + 1]);
      }
    }
  }
  __syncthreads();
  for (int item = tid; item < n_heads * 2 * PER; item += DP_THREADS) {
    const int r = item / (2 * PER), rest = item % (2 * PER), mp = rest / PER, c = rest % PER;
    float big = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) big = fmaxf(big, meet[((w * 2 + mp) * 16 + r) * MPER]);
    float value;
    if (c == 0) {
      value = big;
    } else {
      value = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float* src = meet + ((w * 2 + mp) * 16 + r) * MPER;
        const float f = src[0] == -INFINITY ? 0.f : exp2f(src[0] - big);
        value += src[c] * f;
      }
    }
    if (CLUSTER) own[(r * 2 + mp) * PER + c] = value;
    else mine[(size_t)r * n_splits * 2 * PER + mp * PER + c] = value;
  }
  TL(5);
  if (CLUSTER) {
    SB_BEHIND_WAIT(gate);
    diff_decode_cluster_finish<VD>(own, split, n_splits, n_heads, row, heads, head0, gate, gate_stride, out, tail);
  }
  TL(6);
#ifdef DD_TIMELINE
  if (tid == 0 && part) {
    unsigned long long* dst = reinterpret_cast<unsigned long long*>(part) +
        ((size_t)(blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 8;
    for (int k = 0; k < 7; ++k) dst[k] = tl[k];
    unsigned int sm;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
    dst[7] = sm;
  }
#endif
}

// Joins the parts of one (row, head) and finishes the head.  part: [rows][heads][n_splits][2][v_dim + 2]
// = (maximum in the base-2 domain, sum, accumulator) per map.
__global__ void diff_decode_merge_kernel(const float* __restrict__ part, const bf16* __restrict__ gate, int gate_stride,
                                         bf16* __restrict__ out, int heads, int v_dim, int n_splits,
                                         DiffPrefillTail tail) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(part);
  SB_BEHIND_WAIT(gate);
  const int row = blockIdx.x / heads, head = blockIdx.x % heads;
  const int per = v_dim + 2;
  const float* src = part + ((size_t)row * heads + head) * n_splits * 2 * per;
  float big[2] = {-INFINITY, -INFINITY};
  for (int s = 0; s < n_splits; ++s) {
    big[0] = fmaxf(big[0], src[(size_t)s * 2 * per]);
    big[1] = fmaxf(big[1], src[(size_t)s * 2 * per + per]);
  }
  float den[2] = {0.f, 0.f};
  for (int s = 0; s < n_splits; ++s)
    for (int mp = 0; mp < 2; ++mp) {
      const float m = src[(size_t)s * 2 * per + mp * per];
      if (m != -INFINITY) den[mp] += src[(size_t)s * 2 * per + mp * per + 1] * exp2f(m - big[mp]);
    }
  float mine[2] = {0.f, 0.f};      // up to two columns a thread (v_dim <= 2 * blockDim)
  float ss = 0.f;
  for (int i = 0, c = threadIdx.x; c < v_dim; c += blockDim.x, ++i) {
    float a[2] = {0.f, 0.f};
    for (int s = 0; s < n_splits; ++s)
      for (int mp = 0; mp < 2; ++mp) {
        const float m = src[(size_t)s * 2 * per + mp * per];
        if (m != -INFINITY) a[mp] += src[(size_t)s * 2 * per + mp * per + 2 + c] * exp2f(m - big[mp]);
      }
    const float d = a[0] / den[0] - tail.lambda * (a[1] / den[1]);
    if (i < 2) mine[i] = d;
    ss += d * d;
  }
  ss = block_sum(ss, scratch);
  const float norm = rsqrtf(ss / (float)v_dim + tail.eps) * tail.out_scale;
  for (int i = 0, c = threadIdx.x; c < v_dim; c += blockDim.x, ++i) {
    float v = mine[i] * norm;
    if (gate) v *= 1.f / (1.f + __expf(-__bfloat162float(gate[(size_t)row * gate_stride + (size_t)head * v_dim + c])));
    out[((size_t)row * heads + head) * v_dim + c] = __float2bfloat16_rn(v);
  }
}

// *finished: the one launch also finished the heads (the parts are a cluster); otherwise the parts are
// in `part` and the merge kernel must follow.
template <int QK, int VD>
static int launch_decode(const void* q, const void* k_store, const void* v_store, const int* block_table,
                         int table_stride, const int* row_slot, const int* row_kv_len, int rows, int heads,
                         int kv_heads, float scale, int window, int n_splits, float* part, int early,
                         const void* gate, int gate_stride, void* out, DiffPrefillTail tail, int cluster,
                         bool* finished, cudaStream_t s) {
  constexpr int ring = DD_STAGES * SB_PAGE_TOKENS * (QK + VD) * 2;
  constexpr int meeting = 4 * 2 * 16 * (VD + 8) * 4 + 16 * 2 * (VD + 2) * 4;   // the warps' results, the block's part
  const int smem = 16 * QK * 2 + (ring > meeting ? ring : meeting);     // the meeting area lies over the ring
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(diff_decode_kernel<QK, VD, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(diff_decode_kernel<QK, VD, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int chunks = (heads / kv_heads + 15) / 16;
  const dim3 grid(n_splits, kv_heads * chunks, rows);
  *finished = cluster && n_splits <= DD_CLUSTER_MAX;
  if (*finished)
    return launch_dependent_cluster(diff_decode_kernel<QK, VD, true>, grid, dim3(DP_THREADS), smem, s,
        dim3(n_splits, 1, 1), (const bf16*)q, (const bf16*)k_store, (const bf16*)v_store, block_table, table_stride,
        row_slot, row_kv_len, heads, kv_heads, scale * 1.4426950408889634f, window, n_splits, part, early,
        (const bf16*)gate, gate_stride, (bf16*)out, tail);
  return launch_dependent(diff_decode_kernel<QK, VD, false>, grid, dim3(DP_THREADS), smem, s,
      (const bf16*)q, (const bf16*)k_store, (const bf16*)v_store, block_table, table_stride, row_slot, row_kv_len,
      heads, kv_heads, scale * 1.4426950408889634f, window, n_splits, part, early, (const bf16*)gate, gate_stride,
      (bf16*)out, tail);
}

template <int QK, int VD>
static int launch(const void* q, const void* gate, int gate_stride, void* out, const void* k_store,
                  const void* v_store, const int* block_table, int table_stride, const int* seq_slot,
                  const int* seq_q_start, const int* seq_q_len, const int* seq_kv_len, const int* tile_seq,
                  const int* tile_first, int n_tiles, int heads, int kv_heads, float scale, int window,
                  DiffPrefillTail tail, cudaStream_t s) {
  const int smem = DP_BQ * QK * 2 + 2 * SB_PAGE_TOKENS * (QK + VD) * 2;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(diff_prefill_kernel<QK, VD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return launch_dependent(diff_prefill_kernel<QK, VD>, dim3(n_tiles, heads), dim3(DP_THREADS), smem, s,
      (const bf16*)q, (const bf16*)gate, gate_stride, (bf16*)out, (const bf16*)k_store, (const bf16*)v_store,
      block_table, table_stride, seq_slot, seq_q_start, seq_q_len, seq_kv_len, tile_seq, tile_first, heads,
      kv_heads, scale * 1.4426950408889634f, window, tail);
}

extern "C" {

// 1 if the kernel is built for these sizes.
int sb_diff_prefill_takes(int dim, int v_dim) {
  return (dim == 16 || dim == 32 || dim == 64 || dim == 128) && (v_dim == 32 || v_dim == 64 || v_dim == 128) &&
         !(dim == 128 && v_dim == 32);
}

// q [tokens, heads * 2 * dim] bfloat16 packed by sequence; gate null or rows of gate_stride elements
// (even, 4-byte aligned) whose first heads * v_dim are the gate's pre-activations; out
// [tokens, heads * v_dim].  The seq_* arrays and the work list of 64-query tiles as in the single-map
// prompt kernel.  Returns -2 for sizes it is not built for.
int sb_diff_prefill(const void* q, const void* gate, int gate_stride, void* out, const void* k_store,
                    const void* v_store, const int* block_table, int table_stride, const int* seq_slot,
                    const int* seq_q_start, const int* seq_q_len, const int* seq_kv_len, const int* tile_seq,
                    const int* tile_first, int n_tiles, int heads, int kv_heads, int dim, int v_dim, float scale,
                    int window, float lambda, float out_scale, float eps, cudaStream_t s) {
  if (n_tiles == 0) return 0;
  if (kv_heads <= 0 || heads % kv_heads || !sb_diff_prefill_takes(dim, v_dim)) return -2;
  if (gate && ((gate_stride & 1) || ((uintptr_t)gate & 3))) return -2;
  DiffPrefillTail tail = {lambda, out_scale, eps};
#define ARGS q, gate, gate_stride, out, k_store, v_store, block_table, table_stride, seq_slot, seq_q_start, \
             seq_q_len, seq_kv_len, tile_seq, tile_first, n_tiles, heads, kv_heads, scale, window, tail, s
#define BY_V(QK) switch (v_dim) { case 32: return launch<QK, 32>(ARGS); case 64: return launch<QK, 64>(ARGS); \
                                  case 128: return launch<QK, 128>(ARGS); default: return -2; }
  switch (dim) {
    case 16: BY_V(32)
    case 32: BY_V(64)
    case 64: BY_V(128)
    case 128:
      if (v_dim == 64) return launch<256, 64>(ARGS);
      if (v_dim == 128) return launch<256, 128>(ARGS);
      return -2;
    default: return -2;
  }
#undef BY_V
#undef ARGS
}

// One query row per sequence (its newest token, already in the cache): q [rows, heads * 2 * dim], out
// [rows, heads * v_dim]; row_kv_len[r] counts the row's own key.  part: float scratch of
// rows * heads * n_splits * 2 * (v_dim + 2), used with more than 8 parts or with cluster == 0: then two
// launches (the walk, the merge), otherwise one (the parts are a thread-block cluster).  early: see the
// kernel.  Returns 0, or 1 when it took two launches.
int sb_diff_decode(const void* q, const void* gate, int gate_stride, void* out, const void* k_store,
                   const void* v_store, const int* block_table, int table_stride, const int* row_slot,
                   const int* row_kv_len, int rows, int heads, int kv_heads, int dim, int v_dim, float scale,
                   int window, float lambda, float out_scale, float eps, int n_splits, float* part, int early,
                   int cluster, cudaStream_t s) {
  if (rows == 0) return 0;
  if (kv_heads <= 0 || heads % kv_heads || !sb_diff_prefill_takes(dim, v_dim) || n_splits < 1 || n_splits > 65535) return -2;
  int rc = -2;
  bool finished = false;
  DiffPrefillTail tail = {lambda, out_scale, eps};
#define ARGS q, k_store, v_store, block_table, table_stride, row_slot, row_kv_len, rows, heads, kv_heads, scale, window, \
             n_splits, part, early, gate, gate_stride, out, tail, cluster, &finished, s
#define BY_V(QK) switch (v_dim) { case 32: rc = launch_decode<QK, 32>(ARGS); break; case 64: rc = launch_decode<QK, 64>(ARGS); break; \
                                  case 128: rc = launch_decode<QK, 128>(ARGS); break; default: return -2; } break;
  switch (dim) {
    case 16: BY_V(32)
    case 32: BY_V(64)
    case 64: BY_V(128)
    case 128:
      if (v_dim == 64) rc = launch_decode<256, 64>(ARGS);
      else if (v_dim == 128) rc = launch_decode<256, 128>(ARGS);
      else return -2;
      break;
    default: return -2;
  }
#undef BY_V
#undef ARGS
  if (rc != 0) return rc > 0 ? rc + 1 : rc;      // a CUDA error code, kept apart from "two launches"
  if (finished) return 0;
  const int threads = v_dim >= 128 ? 128 : 64;
  rc = launch_dependent(diff_decode_merge_kernel, dim3(rows * heads), dim3(threads), 0, s, (const float*)part,
                        (const bf16*)gate, gate_stride, (bf16*)out, heads, v_dim, n_splits, tail);
  return rc == 0 ? 1 : rc > 0 ? rc + 1 : rc;
}

}  // extern "C"
