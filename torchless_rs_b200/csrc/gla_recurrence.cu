// Gated linear attention: a matrix state per head that decays per key channel.
// Per head, with q, k, alpha of `dim` channels and v of `vdim` channels,
//   S_t = diag(alpha_t) S_(t-1) + k_t v_t^T          (S: [dim, vdim], rows belong to key channels)
//   o_t = S_t^T (q_t * q_scale)
//   alpha = sigmoid(za + bias)^(1 / tau) = exp(log_sigmoid(za + bias) / tau)
// where q, k, v and za are the 32-bit outputs of the projections.  The state is 32-bit, lives in a
// per-sequence slot and is carried from step to step; the decay, its logarithm, the state and all
// sums are 32-bit.
//
// The columns of S are independent of one another, so the work is spread over (sequence, head,
// group of columns); a warp owns GLA_COLS columns, its lanes share the rows (row i = lane + 32 r),
// and the tokens of a sequence are walked in order, GLA_PF at a time so that their loads and the
// transcendental work of their decays are in flight together.
//
// These kernels run long, so they let the kernel after them go (programmatic dependent launch) only when
// their main loop is done: a dependent grid that is let go at once sits on the SMs waiting, and its many
// warps took half of the issue slots from a recurrence's few (the four kernels of a long step took 350 us
// in sequence against 177 us each alone, and take 165 us this way).
#include "common.cuh"

#define GLA_COLS 4
#define GLA_WARPS 4
#define GLA_MAX_R 8          // rows per lane: states of up to 256 rows

__device__ __forceinline__ float log_sigmoid(float x) {
  // min(x, 0) - log(1 + exp(-|x|)): no overflow on either side
  return fminf(x, 0.0f) - log1pf(expf(-fabsf(x)));
}

// Lane 8 k (k = 0..3) ends with the sum over the warp of column k (6 shuffles for 4 columns).
__device__ __forceinline__ float gla_warp_sum4(const float (&part)[GLA_COLS], int lane) {
  const bool hi = lane & 16;
  float k0 = hi ? part[2] : part[0], k1 = hi ? part[3] : part[1];
  k0 += __shfl_xor_sync(0xffffffffu, hi ? part[0] : part[2], 16);
  k1 += __shfl_xor_sync(0xffffffffu, hi ? part[1] : part[3], 16);
  const bool b = lane & 8;
  float k = b ? k1 : k0;
  k += __shfl_xor_sync(0xffffffffu, b ? k0 : k1, 8);
  k += __shfl_xor_sync(0xffffffffu, k, 4);
  k += __shfl_xor_sync(0xffffffffu, k, 2);
  k += __shfl_xor_sync(0xffffffffu, k, 1);
  return k;
}

// The decays of all tokens at once, in place: za <- alpha.  For steps of many tokens per sequence,
// so that the sequential walk is left with the recurrence alone.
__global__ void gla_decay_kernel(float* __restrict__ za, int lda, const float* __restrict__ bias, float inv_tau,
                                 int T, int hd) {
  pdl_wait();
  const size_t total = (size_t)T * hd;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / hd;
    const int i = (int)(idx - t * hd);
    const float z = za[t * lda + i] + (bias != nullptr ? bias[i] : 0.0f);
    za[t * lda + i] = expf(log_sigmoid(z) * inv_tau);
  }
}

// PRE: `za` already holds alpha (gla_decay_kernel ran).
template <int R, bool PRE>
__global__ void __launch_bounds__(GLA_WARPS * 32)
gla_scan_kernel(const float* __restrict__ zq, const float* __restrict__ zk, const float* __restrict__ zv, int ld,
                const float* __restrict__ za, int lda, const float* __restrict__ bias, float inv_tau,
                float q_scale, float* __restrict__ state, float* __restrict__ o, int ldo,
                const int* __restrict__ seq_start, const int* __restrict__ seq_slot, int heads, int dim,
                int vdim) {
  pdl_wait();
  const int b = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = (blockIdx.z * GLA_WARPS + warp) * GLA_COLS;
  if (c0 >= vdim) return;
  const int t0 = seq_start[b], t1 = seq_start[b + 1];
  float* S = state + (((size_t)seq_slot[b] * heads + h) * dim) * vdim;
  float s[R][GLA_COLS];
  float bi[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = lane + 32 * r;
    bi[r] = (i < dim && bias != nullptr) ? bias[h * dim + i] : 0.0f;
#pragma unroll
    for (int c = 0; c < GLA_COLS; ++c)
      s[r][c] = (i < dim && c0 + c < vdim) ? S[(size_t)i * vdim + c0 + c] : 0.0f;
  }
  constexpr int PF = R <= 4 ? 8 : 4;
  for (int tb = t0; tb < t1; tb += PF) {
    float qv[PF][R], kv[PF][R], av[PF][R], vv[PF][GLA_COLS];
#pragma unroll
    for (int p = 0; p < PF; ++p) {
      const int t = tb + p < t1 ? tb + p : t1 - 1;
      const float* rq = zq + (size_t)t * ld + h * dim;
      const float* rk = zk + (size_t)t * ld + h * dim;
      const float* ra = za + (size_t)t * lda + h * dim;
      const float* rv = zv + (size_t)t * ld + h * vdim + c0;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int i = lane + 32 * r;
        qv[p][r] = i < dim ? rq[i] * q_scale : 0.0f;
        kv[p][r] = i < dim ? rk[i] : 0.0f;
        av[p][r] = i < dim ? ra[i] : 0.0f;
      }
#pragma unroll
      for (int c = 0; c < GLA_COLS; ++c) vv[p][c] = c0 + c < vdim ? rv[c] : 0.0f;
    }
    if (!PRE) {
#pragma unroll
      for (int p = 0; p < PF; ++p)
        if (tb + p < t1) {
#pragma unroll
          for (int r = 0; r < R; ++r) av[p][r] = expf(log_sigmoid(av[p][r] + bi[r]) * inv_tau);
        }
    }
#pragma unroll
    for (int p = 0; p < PF; ++p) {
      if (tb + p < t1) {
        float part[GLA_COLS];
#pragma unroll
        for (int c = 0; c < GLA_COLS; ++c) part[c] = 0.0f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          if (lane + 32 * r < dim) {
            const float a = av[p][r], k = kv[p][r];
#pragma unroll
            for (int c = 0; c < GLA_COLS; ++c) {
              s[r][c] = fmaf(a, s[r][c], k * vv[p][c]);
              part[c] = fmaf(s[r][c], qv[p][r], part[c]);
            }
          }
        }
        const float sum = gla_warp_sum4(part, lane);
        const int c = lane >> 3;
        if ((lane & 7) == 0 && c0 + c < vdim) o[(size_t)(tb + p) * ldo + h * vdim + c0 + c] = sum;
      }
    }
  }
  pdl_launch_dependents();   // the next kernel may set up while this one writes its results
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = lane + 32 * r;
#pragma unroll
    for (int c = 0; c < GLA_COLS; ++c)
      if (i < dim && c0 + c < vdim) S[(size_t)i * vdim + c0 + c] = s[r][c];
  }
}

// ---------------------------------------------------------------------------------------------------
// Long steps: the same recurrence in three passes, so that a prompt's tokens are not walked one after the
// other by a handful of warps.  A sequence's tokens of the step are cut into chunks of GLA_CHUNK.
//   1. every chunk alone, from a zero state (all chunks at once): local outputs
//        o_t = sum over j <= t in the chunk of ((q_t . prod_{j < i <= t} alpha_i) . k_j) v_j,
//      the chunk's end state E_c, and for every token the decay since the chunk's start A_t = prod alpha.
//   2. per sequence, chunk after chunk (few steps): the state at each chunk's start,
//        S_c = A_last(c-1) . S_(c-1) + E_(c-1),  S_0 = the state in the sequence's slot;
//      the state after the last chunk goes back to the slot.
//   3. every chunk again (all at once): o_t += S_c^T (q_t . A_t).
// The sums are those of the token-by-token walk in another order; everything stays 32-bit, and no
// quotient of decays is formed (A_t <= 1 only ever multiplies).
// ---------------------------------------------------------------------------------------------------
#define GLA_CHUNK 64

// (sequence, first token, token count) of chunk `id`, counted over the step's sequences in order
__device__ __forceinline__ bool gla_find_chunk(int id, const int* seq_start, int B, int* b_out, int* t0, int* n) {
  for (int b = 0; b < B; ++b) {
    const int cnt = seq_start[b + 1] - seq_start[b];
    const int chunks = (cnt + GLA_CHUNK - 1) / GLA_CHUNK;
    if (id < chunks) {
      *b_out = b;
      *t0 = seq_start[b] + id * GLA_CHUNK;
      const int left = seq_start[b + 1] - *t0;
      *n = left < GLA_CHUNK ? left : GLA_CHUNK;
      return true;
    }
    id -= chunks;
  }
  return false;
}

// Pass 1.  `za` holds the decays alpha.  ends: [chunks][heads][dim][vdim]; cum: [T][heads * dim].
template <int R>
__global__ void __launch_bounds__(GLA_WARPS * 32)
gla_chunk_local_kernel(const float* __restrict__ zq, const float* __restrict__ zk, const float* __restrict__ zv, int ld,
                       const float* __restrict__ za, int lda, float q_scale, float* __restrict__ ends,
                       float* __restrict__ cum, float* __restrict__ o, int ldo, const int* __restrict__ seq_start,
                       int B, int heads, int dim, int vdim) {
  pdl_wait();
  const int h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = (blockIdx.z * GLA_WARPS + warp) * GLA_COLS;
  int b, t0, n;
  if (!gla_find_chunk(blockIdx.x, seq_start, B, &b, &t0, &n)) return;
  if (c0 >= vdim) return;
  const bool writes_cum = blockIdx.z == 0 && warp == 0;
  float s[R][GLA_COLS], run[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    run[r] = 1.0f;
#pragma unroll
    for (int c = 0; c < GLA_COLS; ++c) s[r][c] = 0.0f;
  }
  constexpr int PF = R <= 4 ? 8 : 4;
  const int t1 = t0 + n;
  for (int tb = t0; tb < t1; tb += PF) {
    float qv[PF][R], kv[PF][R], av[PF][R], vv[PF][GLA_COLS];
#pragma unroll
    for (int p = 0; p < PF; ++p) {
      const int t = tb + p < t1 ? tb + p : t1 - 1;
      const float* rq = zq + (size_t)t * ld + h * dim;
      const float* rk = zk + (size_t)t * ld + h * dim;
      const float* ra = za + (size_t)t * lda + h * dim;
      const float* rv = zv + (size_t)t * ld + h * vdim + c0;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int i = lane + 32 * r;
        qv[p][r] = i < dim ? rq[i] * q_scale : 0.0f;
        kv[p][r] = i < dim ? rk[i] : 0.0f;
        av[p][r] = i < dim ? ra[i] : 0.0f;
      }
#pragma unroll
      for (int c = 0; c < GLA_COLS; ++c) vv[p][c] = c0 + c < vdim ? rv[c] : 0.0f;
    }
#pragma unroll
    for (int p = 0; p < PF; ++p) {
      if (tb + p < t1) {
        float part[GLA_COLS];
#pragma unroll
        for (int c = 0; c < GLA_COLS; ++c) part[c] = 0.0f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          if (lane + 32 * r < dim) {
            const float a = av[p][r], k = kv[p][r];
            run[r] *= a;
            if (writes_cum) cum[(size_t)(tb + p) * heads * dim + h * dim + lane + 32 * r] = run[r];
#pragma unroll
            for (int c = 0; c < GLA_COLS; ++c) {
              s[r][c] = fmaf(a, s[r][c], k * vv[p][c]);
              part[c] = fmaf(s[r][c], qv[p][r], part[c]);
            }
          }
        }
        const float sum = gla_warp_sum4(part, lane);
        const int c = lane >> 3;
        if ((lane & 7) == 0 && c0 + c < vdim) o[(size_t)(tb + p) * ldo + h * vdim + c0 + c] = sum;
      }
    }
  }
  pdl_launch_dependents();   // the next kernel may set up while this one writes its results
  float* E = ends + (((size_t)blockIdx.x * heads + h) * dim) * vdim;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = lane + 32 * r;
#pragma unroll
    for (int c = 0; c < GLA_COLS; ++c)
      if (i < dim && c0 + c < vdim) E[(size_t)i * vdim + c0 + c] = s[r][c];
  }
}

// Pass 1 for states of up to 128 rows: a thread owns one column of the state with all its rows in
// registers, so a token's output is a sum inside the thread (no exchange between lanes) and q, k and
// the decay, which all columns share, are read from shared memory by all lanes at once.  Tokens are
// staged 16 at a time.  Per token and column: `dim` times (one product, two fused multiply-adds).
#define GLA_SUB 16
template <int R>
__global__ void __launch_bounds__(128)
gla_chunk_local_cols_kernel(const float* __restrict__ zq, const float* __restrict__ zk, const float* __restrict__ zv,
                            int ld, const float* __restrict__ za, int lda, float q_scale, float* __restrict__ ends,
                            float* __restrict__ cum, float* __restrict__ o, int ldo,
                            const int* __restrict__ seq_start, int B, int heads, int dim, int vdim) {
  constexpr int D = 32 * R;                    // rows held (dim rounded up; the rest are zero)
  __shared__ __align__(16) float sq[GLA_SUB][D], sk[GLA_SUB][D], sa[GLA_SUB][D];
  pdl_wait();
  const int h = blockIdx.y, tid = threadIdx.x;
  const int c = blockIdx.z * 128 + tid;
  int b, t0, n;
  if (!gla_find_chunk(blockIdx.x, seq_start, B, &b, &t0, &n)) return;
  float s[D];
#pragma unroll
  for (int i = 0; i < D; ++i) s[i] = 0.0f;
  float run = 1.0f;                            // thread i < dim: the decay of row i since the chunk's start
  for (int tb = 0; tb < n; tb += GLA_SUB) {
    const int cnt = n - tb < GLA_SUB ? n - tb : GLA_SUB;
    __syncthreads();
    for (int idx = tid; idx < GLA_SUB * D; idx += 128) {
      const int p = idx / D, i = idx - p * D;
      const bool ok = p < cnt && i < dim;
      const size_t t = t0 + tb + p;
      sq[p][i] = ok ? zq[t * ld + h * dim + i] * q_scale : 0.0f;
      sk[p][i] = ok ? zk[t * ld + h * dim + i] : 0.0f;
      sa[p][i] = ok ? za[t * lda + h * dim + i] : 0.0f;
    }
    float vv[GLA_SUB];
#pragma unroll
    for (int p = 0; p < GLA_SUB; ++p)
      vv[p] = (p < cnt && c < vdim) ? zv[(size_t)(t0 + tb + p) * ld + h * vdim + c] : 0.0f;
    __syncthreads();
    if (blockIdx.z == 0 && tid < dim) {
      for (int p = 0; p < cnt; ++p) {
        run *= sa[p][tid];
        cum[(size_t)(t0 + tb + p) * heads * dim + h * dim + tid] = run;
      }
    }
#pragma unroll
    for (int p = 0; p < GLA_SUB; ++p) {
      if (p >= cnt) continue;
      const float v = vv[p];
      float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll
      for (int i = 0; i < D; i += 4) {
        const float4 a4 = *reinterpret_cast<const float4*>(&sa[p][i]);
        const float4 k4 = *reinterpret_cast<const float4*>(&sk[p][i]);
        const float4 q4 = *reinterpret_cast<const float4*>(&sq[p][i]);
        s[i] = fmaf(a4.x, s[i], k4.x * v);
        s[i + 1] = fmaf(a4.y, s[i + 1], k4.y * v);
        s[i + 2] = fmaf(a4.z, s[i + 2], k4.z * v);
        s[i + 3] = fmaf(a4.w, s[i + 3], k4.w * v);
        acc0 = fmaf(s[i], q4.x, acc0);
        acc1 = fmaf(s[i + 1], q4.y, acc1);
        acc0 = fmaf(s[i + 2], q4.z, acc0);
        acc1 = fmaf(s[i + 3], q4.w, acc1);
      }
      if (c < vdim) o[(size_t)(t0 + tb + p) * ldo + h * vdim + c] = acc0 + acc1;
    }
  }
  pdl_launch_dependents();   // the next kernel may set up while this one writes its results
  if (c < vdim) {
    float* E = ends + (((size_t)blockIdx.x * heads + h) * dim) * vdim + c;
#pragma unroll
    for (int i = 0; i < D; ++i)
      if (i < dim) E[(size_t)i * vdim] = s[i];
  }
}

// Pass 2.  starts: [chunks][heads][dim][vdim] receives the state at each chunk's start.
template <int R>
__global__ void __launch_bounds__(GLA_WARPS * 32)
gla_chunk_carry_kernel(const float* __restrict__ ends, const float* __restrict__ cum, float* __restrict__ starts,
                       float* __restrict__ state, const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                       int heads, int dim, int vdim) {
  pdl_wait();
  const int b = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = (blockIdx.z * GLA_WARPS + warp) * GLA_COLS;
  if (c0 >= vdim) return;
  int chunk = 0;
  for (int i = 0; i < b; ++i) chunk += (seq_start[i + 1] - seq_start[i] + GLA_CHUNK - 1) / GLA_CHUNK;
  const int t_begin = seq_start[b], t_end = seq_start[b + 1];
  float* S = state + (((size_t)seq_slot[b] * heads + h) * dim) * vdim;
  float s[R][GLA_COLS];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = lane + 32 * r;
#pragma unroll
    for (int c = 0; c < GLA_COLS; ++c)
      s[r][c] = (i < dim && c0 + c < vdim) ? S[(size_t)i * vdim + c0 + c] : 0.0f;
  }
  // the end state and decay of a chunk are fetched while the chunk before it is folded in
  float e_next[R][GLA_COLS], d_next[R];
  auto fetch = [&](int t0, int ch) {
    const int last = (t0 + GLA_CHUNK < t_end ? t0 + GLA_CHUNK : t_end) - 1;
    const size_t base = (((size_t)ch * heads + h) * dim) * vdim;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int i = lane + 32 * r;
      d_next[r] = i < dim ? cum[(size_t)last * heads * dim + h * dim + i] : 0.0f;
#pragma unroll
      for (int c = 0; c < GLA_COLS; ++c)
        e_next[r][c] = (i < dim && c0 + c < vdim) ? ends[base + (size_t)i * vdim + c0 + c] : 0.0f;
    }
  };
  if (t_begin < t_end) fetch(t_begin, chunk);
  for (int t0 = t_begin; t0 < t_end; t0 += GLA_CHUNK, ++chunk) {
    const size_t base = (((size_t)chunk * heads + h) * dim) * vdim;
    float e[R][GLA_COLS], d[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      d[r] = d_next[r];
#pragma unroll
      for (int c = 0; c < GLA_COLS; ++c) e[r][c] = e_next[r][c];
    }
    if (t0 + GLA_CHUNK < t_end) fetch(t0 + GLA_CHUNK, chunk + 1);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int i = lane + 32 * r;
      if (i >= dim) continue;
#pragma unroll
      for (int c = 0; c < GLA_COLS; ++c)
        if (c0 + c < vdim) {
          starts[base + (size_t)i * vdim + c0 + c] = s[r][c];
          s[r][c] = fmaf(d[r], s[r][c], e[r][c]);
        }
    }
  }
  pdl_launch_dependents();   // the next kernel may set up while this one writes its results
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = lane + 32 * r;
#pragma unroll
    for (int c = 0; c < GLA_COLS; ++c)
      if (i < dim && c0 + c < vdim) S[(size_t)i * vdim + c0 + c] = s[r][c];
  }
}

// Pass 3: o[t, h, n] += sum_i (q[t, i] * q_scale * cum[t, i]) * starts[chunk][h][i][n], a 64 x dim by
// dim x 64 product per block on CUDA cores (16 x 16 threads, 4 x 4 outputs each).
__global__ void __launch_bounds__(256)
gla_chunk_apply_kernel(const float* __restrict__ zq, int ld, const float* __restrict__ cum, float q_scale,
                       const float* __restrict__ starts, float* __restrict__ o, int ldo,
                       const int* __restrict__ seq_start, int B, int heads, int dim, int vdim) {
  __shared__ float As[16][GLA_CHUNK + 4];
  __shared__ float Bs[16][64 + 4];
  pdl_wait();
  const int h = blockIdx.y, n0 = blockIdx.z * 64, tid = threadIdx.x;
  int b, t0, n;
  if (!gla_find_chunk(blockIdx.x, seq_start, B, &b, &t0, &n)) return;
  const float* Sc = starts + (((size_t)blockIdx.x * heads + h) * dim) * vdim;
  const int tx = tid & 15, ty = tid >> 4;
  float acc[4][4] = {};
  const int lrow = tid >> 2, lk = (tid & 3) * 4;     // A: 64 tokens x 16 i, four i per thread
  const int brow = tid >> 4, bcol = (tid & 15) * 4;  // B: 16 i x 64 columns, four columns per thread
  for (int k0 = 0; k0 < dim; k0 += 16) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = k0 + lk + j, t = t0 + lrow;
      As[lk + j][lrow] = (lrow < n && i < dim)
          ? zq[(size_t)t * ld + h * dim + i] * q_scale * cum[(size_t)t * heads * dim + h * dim + i] : 0.0f;
      const int bi = k0 + brow, col = n0 + bcol + j;
      Bs[brow][bcol + j] = (bi < dim && col < vdim) ? Sc[(size_t)bi * vdim + col] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Bs[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
  pdl_launch_dependents();   // the next kernel may set up while this one writes its results
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = ty * 4 + i;
    if (m >= n) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = n0 + tx * 4 + j;
      if (col < vdim) o[(size_t)(t0 + m) * ldo + h * vdim + col] += acc[i][j];
    }
  }
}

// Floats of scratch that a step of T tokens of B sequences needs for the three passes (0: the step is
// walked token by token).  Long steps only: the passes cost three launches and twice the state per chunk.
extern "C" long long TL_NAME(tl_gla_scan_scratch)(int T, int B, int heads, int dim, int vdim) {
  if (T < 4 * GLA_CHUNK || T <= 4 * B) return 0;
  const long long chunks = T / GLA_CHUNK + B;
  return 2 * chunks * heads * dim * vdim + (long long)T * heads * dim;
}

// zq, zk, zv: columns of one 32-bit product [T, ld]; za: [T, lda] 32-bit pre-activations of the decay
// (overwritten with the decays when the step has many tokens per sequence, T > 4 B), or, with `given`,
// the decays themselves, which are only read (lda may then be 0: one row of decays for every token, a
// recurrence whose decay is a constant of the head); bias:
// [heads * dim] or null; state: [slots, heads, dim, vdim]; o: [T, ldo]; sequence b owns the tokens
// seq_start[b] .. seq_start[b + 1] - 1 of the step.
extern "C" int TL_NAME(tl_gla_scan)(const float* zq, const float* zk, const float* zv, int ld, float* za, int lda,
                                    const float* bias, float tau, float q_scale, float* state, float* o, int ldo,
                                    const int* seq_start, const int* seq_slot, int T, int B, int heads, int dim,
                                    int vdim, float* scratch, int given, cudaStream_t stream) {
  if (B <= 0 || T <= 0) return 0;
  if (heads <= 0 || dim <= 0 || vdim <= 0 || (!given && !(tau > 0.0f))) return TL_ERR_BAD_ARG;
  const int R = (dim + 31) / 32;
  if (heads > 65535 || R > GLA_MAX_R) return TL_ERR_UNSUPPORTED;
  const int per_block = GLA_WARPS * GLA_COLS;
  dim3 grid(B, heads, (vdim + per_block - 1) / per_block);
  if (grid.z > 65535) return TL_ERR_UNSUPPORTED;
  const float inv_tau = given ? 1.0f : 1.0f / tau;
  const bool pre = given || T > 4 * B;
  if (pre && !given) {
    const size_t total = (size_t)T * heads * dim;
    const unsigned blocks = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    const int rc = tl_launch(gla_decay_kernel, dim3(blocks), dim3(256), 0, stream, za, lda, bias, inv_tau, T,
                             heads * dim);
    if (rc != 0) return rc;
  }
  if (scratch != nullptr && TL_NAME(tl_gla_scan_scratch)(T, B, heads, dim, vdim) > 0) {
    // the three passes; `za` holds the decays by now
    const int chunks = T / GLA_CHUNK + B;
    const size_t per = (size_t)chunks * heads * dim * vdim;
    float *ends = scratch, *starts = scratch + per, *cum = scratch + 2 * per;
    dim3 g1(chunks, heads, grid.z);
    int rc3;
    if (R <= 4) {
      // a column per thread
      dim3 gc(chunks, heads, (vdim + 127) / 128);
#define COLS(RR)                                                                                              \
      rc3 = tl_launch(gla_chunk_local_cols_kernel<RR>, gc, dim3(128), 0, stream, zq, zk, zv, ld,              \
                      (const float*)za, lda, q_scale, ends, cum, o, ldo, seq_start, B, heads, dim, vdim);     \
      if (rc3 == 0)                                                                                           \
        rc3 = tl_launch(gla_chunk_carry_kernel<RR>, grid, dim3(GLA_WARPS * 32), 0, stream, (const float*)ends,\
                        (const float*)cum, starts, state, seq_start, seq_slot, heads, dim, vdim);             \
      break
      switch (R) {
        case 1: COLS(1);
        case 2: COLS(2);
        case 3: COLS(3);
        default: COLS(4);
      }
#undef COLS
      if (rc3 != 0) return rc3;
      return tl_launch(gla_chunk_apply_kernel, dim3(chunks, heads, (vdim + 63) / 64), dim3(256), 0, stream, zq, ld,
                       (const float*)cum, q_scale, (const float*)starts, o, ldo, seq_start, B, heads, dim, vdim);
    }
#define CHUNKED(RR)                                                                                           \
    rc3 = tl_launch(gla_chunk_local_kernel<RR>, g1, dim3(GLA_WARPS * 32), 0, stream, zq, zk, zv, ld,          \
                    (const float*)za, lda, q_scale, ends, cum, o, ldo, seq_start, B, heads, dim, vdim);       \
    if (rc3 == 0)                                                                                             \
      rc3 = tl_launch(gla_chunk_carry_kernel<RR>, grid, dim3(GLA_WARPS * 32), 0, stream, (const float*)ends,  \
                      (const float*)cum, starts, state, seq_start, seq_slot, heads, dim, vdim);               \
    break
    switch (R) {
      case 1: CHUNKED(1);
      case 2: CHUNKED(2);
      case 3: CHUNKED(3);
      case 4: CHUNKED(4);
      case 5: CHUNKED(5);
      case 6: CHUNKED(6);
      case 7: CHUNKED(7);
      default: CHUNKED(8);
    }
#undef CHUNKED
    if (rc3 != 0) return rc3;
    return tl_launch(gla_chunk_apply_kernel, dim3(chunks, heads, (vdim + 63) / 64), dim3(256), 0, stream, zq, ld,
                     (const float*)cum, q_scale, (const float*)starts, o, ldo, seq_start, B, heads, dim, vdim);
  }
  int rc;
#define SCAN(RR)                                                                                              \
  rc = pre ? tl_launch(gla_scan_kernel<RR, true>, grid, dim3(GLA_WARPS * 32), 0, stream, zq, zk, zv, ld,      \
                       (const float*)za, lda, bias, inv_tau, q_scale, state, o, ldo, seq_start, seq_slot,     \
                       heads, dim, vdim)                                                                      \
           : tl_launch(gla_scan_kernel<RR, false>, grid, dim3(GLA_WARPS * 32), 0, stream, zq, zk, zv, ld,     \
                       (const float*)za, lda, bias, inv_tau, q_scale, state, o, ldo, seq_start, seq_slot,     \
                       heads, dim, vdim);                                                                     \
  break
  switch (R) {
    case 1: SCAN(1);
    case 2: SCAN(2);
    case 3: SCAN(3);
    case 4: SCAN(4);
    case 5: SCAN(5);
    case 6: SCAN(6);
    case 7: SCAN(7);
    default: SCAN(8);
  }
#undef SCAN
  return rc;
}
