// The gated delta rule: a matrix state per head that decays by one number per token and is corrected
// towards the token's value, fed through short causal convolutions.  Per value head h (which reads the
// query/key head h / (heads / kv_heads)), with q, k of `dim` channels and v of `vdim`:
//   S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q          (S: [dim, vdim])
//   g = exp(-exp(A_log) softplus(za + dt_bias)),  beta = sigmoid(zb)
// q, k, v come out of a convolution over the last `taps` tokens of each channel and a silu; q and k are
// then divided by their length (q also by sqrt(dim)).  State, decay, gates, unit norms and all sums are
// 32-bit.  The state and the convolution's last taps - 1 inputs live in per-sequence slots and are carried
// from step to step, so a prompt may come in any number of pieces.
//
//   delta_prep          the step's projections -> convolved, activated, unit-normed q, k, v; beta, g and
//                       k . q per token (everything the walk needs that does not depend on the state)
//   conv_state_update   the last taps - 1 inputs of every sequence go back to its slot
//   delta_scan          the walk over each sequence's tokens of the step, in order (two layouts: one for
//                       steps of few tokens per sequence, one for many)
// and two small kernels that the design's other mixers use: silu over the columns of a 32-bit product, and
// the weighted sum of mixers that run side by side (each with the bias of its output projection, if any).
//
// The columns of S are independent of one another (column c only needs v_c and the shared q, k, g,
// beta), so the walk is spread over (sequence, head, group of columns); a warp owns DR_COLS columns, its
// lanes share the rows (row i = lane + 32 r).  With s' = g s the token's sums r = s' . k and p = s' . q are
// taken in one pass, then u = beta (v - r), o = p + u (k . q) and s = s' + k u: the read-out after the
// write, without a second pass over the state.
#include "common.cuh"

#define DR_COLS 4
#define DR_WARPS 4
#define DR_MAX_R 8          // rows per lane: states of up to 256 rows
#define DR_MAX_TAPS 16

__device__ __forceinline__ float dr_silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float dr_softplus(float x) { return fmaxf(x, 0.0f) + log1pf(expf(-fabsf(x))); }

// One channel of the convolution for the token with local index j of a sequence whose step starts at row
// t0 of z: sum_i w[i] x(j - (taps - 1 - i)), x taken from the step's rows, or from the slot's kept inputs
// (oldest first) where it lies before the step.
__device__ __forceinline__ float dr_conv(const float* __restrict__ z, int ld, int t0, int j, int c,
                                         const float* __restrict__ w, int taps, const float* __restrict__ kept,
                                         int channels) {
  float acc = 0.0f;
  for (int i = 0; i < taps; ++i) {
    const int jj = j - (taps - 1 - i);
    const float x = jj >= 0 ? z[(size_t)(t0 + jj) * ld + c] : kept[(size_t)(taps - 1 + jj) * channels + c];
    acc = fmaf(w[(size_t)c * taps + i], x, acc);
  }
  return acc;
}

// z: [T, ld] 32-bit, columns [q (G dim) | k (G dim) | v (H vdim) | ... | zb at col_b (H) | za at col_a (H)].
// y: [T, ldy] = [q | k | v] after convolution, silu and unit norms.  gates: [T, 2 H + G] = beta, g, k . q.
// A warp per (token, unit): units 0 .. G-1 are the query/key heads, G .. G+H-1 the value heads.
__global__ void __launch_bounds__(DR_WARPS * 32)
delta_prep_kernel(const float* __restrict__ z, int ld, const float* __restrict__ taps_w, int taps,
                  const float* __restrict__ kept, float* __restrict__ y, int ldy, float* __restrict__ gates,
                  const float* __restrict__ neg_a, const float* __restrict__ dt_bias, int col_b, int col_a,
                  const int* __restrict__ token_seq, const int* __restrict__ seq_start,
                  const int* __restrict__ seq_slot, int G, int H, int dim, int vdim, float unit_eps,
                  float q_scale) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int b = token_seq[t];
  const int t0 = seq_start[b], j = t - t0;
  const int channels = 2 * G * dim + H * vdim;
  const float* mine = kept + (size_t)seq_slot[b] * (taps - 1) * channels;
  for (int unit = blockIdx.y * DR_WARPS + warp; unit < G + H; unit += gridDim.y * DR_WARPS) {
    if (unit < G) {
      const int cq = unit * dim, ck = G * dim + unit * dim;
      float q[DR_MAX_R], k[DR_MAX_R];
      float sq = 0.0f, sk = 0.0f;
#pragma unroll
      for (int r = 0; r < DR_MAX_R; ++r) {
        const int i = lane + 32 * r;
        q[r] = k[r] = 0.0f;
        if (i < dim) {
          q[r] = dr_silu(dr_conv(z, ld, t0, j, cq + i, taps_w, taps, mine, channels));
          k[r] = dr_silu(dr_conv(z, ld, t0, j, ck + i, taps_w, taps, mine, channels));
        }
        sq = fmaf(q[r], q[r], sq);
        sk = fmaf(k[r], k[r], sk);
      }
      sq = warp_sum(sq);
      sk = warp_sum(sk);
      const float fq = q_scale / sqrtf(sq + unit_eps), fk = 1.0f / sqrtf(sk + unit_eps);
      float kq = 0.0f;
#pragma unroll
      for (int r = 0; r < DR_MAX_R; ++r) {
        const int i = lane + 32 * r;
        q[r] *= fq;
        k[r] *= fk;
        kq = fmaf(q[r], k[r], kq);
        if (i < dim) {
          y[(size_t)t * ldy + cq + i] = q[r];
          y[(size_t)t * ldy + ck + i] = k[r];
        }
      }
      kq = warp_sum(kq);
      if (lane == 0) gates[(size_t)t * (2 * H + G) + 2 * H + unit] = kq;
    } else {
      const int h = unit - G;
      const int cv = 2 * G * dim + h * vdim;
      for (int i = lane; i < vdim; i += 32)
        y[(size_t)t * ldy + cv + i] = dr_silu(dr_conv(z, ld, t0, j, cv + i, taps_w, taps, mine, channels));
      if (lane == 0) {
        const float zb = z[(size_t)t * ld + col_b + h], za = z[(size_t)t * ld + col_a + h];
        gates[(size_t)t * (2 * H + G) + h] = 1.0f / (1.0f + expf(-zb));
        gates[(size_t)t * (2 * H + G) + H + h] = expf(neg_a[h] * dr_softplus(za + dt_bias[h]));
      }
    }
  }
}

// kept: [slots, taps - 1, channels], oldest first.  A thread per (sequence, channel) reads what it needs
// before it writes, so a step of fewer tokens than taps - 1 moves the older inputs up.
__global__ void __launch_bounds__(256)
conv_state_update_kernel(const float* __restrict__ z, int ld, float* __restrict__ kept, int taps,
                         const int* __restrict__ seq_start, const int* __restrict__ seq_slot, int channels) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int t0 = seq_start[b], n = seq_start[b + 1] - t0;
  float* mine = kept + (size_t)seq_slot[b] * (taps - 1) * channels;
  float v[DR_MAX_TAPS - 1];
#pragma unroll
  for (int i = 0; i < DR_MAX_TAPS - 1; ++i) {
    v[i] = 0.0f;
    if (i < taps - 1) {
      const int jj = n - (taps - 1) + i;
      v[i] = jj >= 0 ? z[(size_t)(t0 + jj) * ld + c] : mine[(size_t)(taps - 1 + jj) * channels + c];
    }
  }
#pragma unroll
  for (int i = 0; i < DR_MAX_TAPS - 1; ++i)
    if (i < taps - 1) mine[(size_t)i * channels + c] = v[i];
}

// Lane 8 k (k = 0..3) ends with the sum over the warp of column k (6 shuffles for 4 columns).
__device__ __forceinline__ float dr_warp_sum4(const float (&part)[DR_COLS], int lane) {
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

// y: [T, ldy] = [q (G dim) | k (G dim) | v (H vdim)], prepared; gates: [T, 2 H + G]; state: [slots, H, dim,
// vdim]; o: [T, ldo].  Lets the next kernel go only when its loop is done (a grid that waits on the SMs
// takes issue slots from the few warps of a recurrence).
template <int R>
__global__ void __launch_bounds__(DR_WARPS * 32)
delta_scan_kernel(const float* __restrict__ y, int ldy, const float* __restrict__ gates,
                  float* __restrict__ state, float* __restrict__ o, int ldo, const int* __restrict__ seq_start,
                  const int* __restrict__ seq_slot, int G, int H, int dim, int vdim) {
  pdl_wait();
  const int b = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = (blockIdx.z * DR_WARPS + warp) * DR_COLS;
  if (c0 >= vdim) return;
  const int g = h / (H / G);
  const int t0 = seq_start[b], t1 = seq_start[b + 1];
  float* S = state + (((size_t)seq_slot[b] * H + h) * dim) * vdim;
  float s[R][DR_COLS];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = lane + 32 * r;
#pragma unroll
    for (int c = 0; c < DR_COLS; ++c)
      s[r][c] = (i < dim && c0 + c < vdim) ? S[(size_t)i * vdim + c0 + c] : 0.0f;
  }
  const int gw = 2 * H + G;
  constexpr int PF = R <= 4 ? 8 : 4;
  for (int tb = t0; tb < t1; tb += PF) {
    float qv[PF][R], kv[PF][R], vv[PF][DR_COLS], beta[PF], dec[PF], kq[PF];
#pragma unroll
    for (int p = 0; p < PF; ++p) {
      const int t = tb + p < t1 ? tb + p : t1 - 1;
      const float* row = y + (size_t)t * ldy;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int i = lane + 32 * r;
        qv[p][r] = i < dim ? row[g * dim + i] : 0.0f;
        kv[p][r] = i < dim ? row[(G + g) * dim + i] : 0.0f;
      }
#pragma unroll
      for (int c = 0; c < DR_COLS; ++c) vv[p][c] = c0 + c < vdim ? row[2 * G * dim + h * vdim + c0 + c] : 0.0f;
      beta[p] = gates[(size_t)t * gw + h];
      dec[p] = gates[(size_t)t * gw + H + h];
      kq[p] = gates[(size_t)t * gw + 2 * H + g];
    }
#pragma unroll
    for (int p = 0; p < PF; ++p) {
      if (tb + p < t1) {
        float pr[DR_COLS], pp[DR_COLS];
#pragma unroll
        for (int c = 0; c < DR_COLS; ++c) pr[c] = pp[c] = 0.0f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
          for (int c = 0; c < DR_COLS; ++c) {
            s[r][c] *= dec[p];
            pr[c] = fmaf(s[r][c], kv[p][r], pr[c]);
            pp[c] = fmaf(s[r][c], qv[p][r], pp[c]);
          }
        }
        const float rs = dr_warp_sum4(pr, lane);      // lane 8 c: column c's s' . k
        const float ps = dr_warp_sum4(pp, lane);      // lane 8 c: column c's s' . q
        const int mc = lane >> 3;
        const float vm = mc == 0 ? vv[p][0] : mc == 1 ? vv[p][1] : mc == 2 ? vv[p][2] : vv[p][3];
        const float um = beta[p] * (vm - rs);          // valid in lanes 0, 8, 16, 24
        if ((lane & 7) == 0 && c0 + mc < vdim) o[(size_t)(tb + p) * ldo + h * vdim + c0 + mc] = fmaf(um, kq[p], ps);
        float u[DR_COLS];
#pragma unroll
        for (int c = 0; c < DR_COLS; ++c) u[c] = __shfl_sync(0xffffffffu, um, 8 * c);
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
          for (int c = 0; c < DR_COLS; ++c) s[r][c] = fmaf(kv[p][r], u[c], s[r][c]);
        }
      }
    }
  }
  pdl_launch_dependents();
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = lane + 32 * r;
#pragma unroll
    for (int c = 0; c < DR_COLS; ++c)
      if (i < dim && c0 + c < vdim) S[(size_t)i * vdim + c0 + c] = s[r][c];
  }
}

// The walk for steps of many tokens.  LPC lanes share a column of the state, each holding ROWS of its rows
// (the 16-byte pieces of a row vector go to the lanes in turn, so that the lanes of a warp read neighbouring
// pieces of shared memory); a warp covers 32 / LPC columns, a block one (sequence, head) and four warps'
// columns.  The tokens' q, k and gates come through shared memory in tiles of DR_TILE tokens, the next tile
// on its way (cp.async) while this one is walked.  A walk has sequences x heads x columns chains that wait
// for nothing but themselves and the GPU has room for more warps than that, so a column is spread over as
// many lanes as leave each lane a piece or two: what a warp executes per token is what the step takes.
#define DR_TILE 16

__device__ __forceinline__ void dr_cp4(float* dst, const float* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}

__device__ __forceinline__ void dr_cp16(float* dst, const float* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}

__device__ __forceinline__ void dr_store_if(float* p, float v, bool yes) {
  asm volatile("{\n .reg .pred q;\n setp.ne.b32 q, %2, 0;\n @q st.global.f32 [%0], %1;\n}" ::"l"(p), "f"(v), "r"((int)yes)
               : "memory");
}

template <int ROWS, int LPC>
__global__ void __launch_bounds__(128)
delta_scan_tiled_kernel(const float* __restrict__ y, int ldy, const float* __restrict__ gates,
                        float* __restrict__ state, float* __restrict__ o, int ldo,
                        const int* __restrict__ seq_start, const int* __restrict__ seq_slot, int G, int H, int dim,
                        int vdim) {
  constexpr int DP = LPC * ROWS;                             // rows, padded
  constexpr int CPW = 32 / LPC;                              // columns of a warp
  __shared__ __align__(16) float kq_s[2][DR_TILE][2 * DP];   // per token: k, then q
  __shared__ __align__(16) float g_s[2][DR_TILE][4];         // per token: beta, decay, k . q
  pdl_wait();
  const int b = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane & (LPC - 1);
  const int col = (blockIdx.z * 4 + warp) * CPW + lane / LPC;
  const bool live = col < vdim;
  const int g = h / (H / G);
  const int t0 = seq_start[b], t1 = seq_start[b + 1];
  const int gw = 2 * H + G;
  float* S = state + (((size_t)seq_slot[b] * H + h) * dim) * vdim;
  // register i = 4 j + e holds row 4 (LPC j + sub) + e
  float s[ROWS];
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int row = 4 * (LPC * (i >> 2) + sub) + (i & 3);
    s[i] = (live && row < dim) ? S[(size_t)row * vdim + col] : 0.0f;
  }
  // rows past `dim` stay zero in both buffers: they are never copied into
  for (int idx = threadIdx.x; idx < 2 * DR_TILE * 2 * DP; idx += blockDim.x) (&kq_s[0][0][0])[idx] = 0.0f;
  __syncthreads();
  const float* yk = y + (size_t)(G + g) * dim;
  const float* yq = y + (size_t)g * dim;
  // eight threads copy one token's k and q, in 16-byte pieces where the rows allow it
  const bool wide = (dim & 3) == 0 && (ldy & 3) == 0 && ((uintptr_t)y & 15) == 0;
  const int ft = threadIdx.x >> 3, fp = threadIdx.x & 7;
  auto fetch = [&](int buf, int tb) {
    const int n = min(DR_TILE, t1 - tb);
    if (ft < n) {
      const float* rk = yk + (size_t)(tb + ft) * ldy;
      const float* rq = yq + (size_t)(tb + ft) * ldy;
      if (wide) {
        for (int i = fp * 4; i < dim; i += 32) {
          dr_cp16(&kq_s[buf][ft][i], rk + i);
          dr_cp16(&kq_s[buf][ft][DP + i], rq + i);
        }
      } else {
        for (int i = fp; i < dim; i += 8) {
          dr_cp4(&kq_s[buf][ft][i], rk + i);
          dr_cp4(&kq_s[buf][ft][DP + i], rq + i);
        }
      }
    }
    if ((int)threadIdx.x < n) {
      const float* gr = gates + (size_t)(tb + threadIdx.x) * gw;
      dr_cp4(&g_s[buf][threadIdx.x][0], gr + h);
      dr_cp4(&g_s[buf][threadIdx.x][1], gr + H + h);
      dr_cp4(&g_s[buf][threadIdx.x][2], gr + 2 * H + g);
    } else if ((int)threadIdx.x < DR_TILE) {
      // a place past the step's end writes nothing (beta 0) and decays nothing, so the walk below needs no
      // branch per token and its loads can run ahead of the token before
      g_s[buf][threadIdx.x][0] = 0.0f;
      g_s[buf][threadIdx.x][1] = 1.0f;
      g_s[buf][threadIdx.x][2] = 0.0f;
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (t0 < t1) fetch(0, t0);
  int buf = 0;
  for (int tb = t0; tb < t1; tb += DR_TILE, buf ^= 1) {
    const int n = min(DR_TILE, t1 - tb);
    if (tb + DR_TILE < t1) {
      fetch(buf ^ 1, tb + DR_TILE);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    float vv[DR_TILE];
#pragma unroll
    for (int tt = 0; tt < DR_TILE; ++tt)
      vv[tt] = (live && tt < n) ? y[(size_t)(tb + tt) * ldy + 2 * G * dim + h * vdim + col] : 0.0f;
    float* o_col = o + (size_t)tb * ldo + h * vdim + (live ? col : 0);
    const bool writes = live && sub == 0;
    __syncthreads();
    // a token's k, q and gates are asked for while the token before is worked on
    float4 k4[ROWS / 4], q4[ROWS / 4], gt;
    {
      const float4* kk = reinterpret_cast<const float4*>(&kq_s[buf][0][0]);
      const float4* qq = reinterpret_cast<const float4*>(&kq_s[buf][0][DP]);
#pragma unroll
      for (int j = 0; j < ROWS / 4; ++j) {
        k4[j] = kk[LPC * j + sub];
        q4[j] = qq[LPC * j + sub];
      }
      gt = *reinterpret_cast<const float4*>(&g_s[buf][0][0]);
    }
#pragma unroll
    for (int tt = 0; tt < DR_TILE; ++tt) {
      float4 k4n[ROWS / 4], q4n[ROWS / 4], gtn;
      if (tt + 1 < DR_TILE) {
        const float4* kk = reinterpret_cast<const float4*>(&kq_s[buf][tt + 1][0]);
        const float4* qq = reinterpret_cast<const float4*>(&kq_s[buf][tt + 1][DP]);
#pragma unroll
        for (int j = 0; j < ROWS / 4; ++j) {
          k4n[j] = kk[LPC * j + sub];
          q4n[j] = qq[LPC * j + sub];
        }
        gtn = *reinterpret_cast<const float4*>(&g_s[buf][tt + 1][0]);
      }
      const float beta = gt.x, dec = gt.y, kq = gt.z;
      float r[4] = {0.0f, 0.0f, 0.0f, 0.0f}, p[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int j = 0; j < ROWS / 4; ++j) {
        r[0] = fmaf(s[4 * j], k4[j].x, r[0]);     p[0] = fmaf(s[4 * j], q4[j].x, p[0]);
        r[1] = fmaf(s[4 * j + 1], k4[j].y, r[1]); p[1] = fmaf(s[4 * j + 1], q4[j].y, p[1]);
        r[2] = fmaf(s[4 * j + 2], k4[j].z, r[2]); p[2] = fmaf(s[4 * j + 2], q4[j].z, p[2]);
        r[3] = fmaf(s[4 * j + 3], k4[j].w, r[3]); p[3] = fmaf(s[4 * j + 3], q4[j].w, p[3]);
      }
      float rs = (r[0] + r[1]) + (r[2] + r[3]), ps = (p[0] + p[1]) + (p[2] + p[3]);
#pragma unroll
      for (int m = 1; m < LPC; m <<= 1) {
        rs += __shfl_xor_sync(0xffffffffu, rs, m);
        ps += __shfl_xor_sync(0xffffffffu, ps, m);
      }
      // the sums were taken over the state before its decay: s' = dec s
      const float u = beta * (vv[tt] - dec * rs);
      // (a store under a predicate, not a branch: the tile stays one straight run of instructions, so the
      // loads of later tokens are scheduled ahead of the tokens before)
      dr_store_if(o_col + (size_t)tt * ldo, fmaf(u, kq, dec * ps), writes && tt < n);
#pragma unroll
      for (int j = 0; j < ROWS / 4; ++j) {
        s[4 * j] = fmaf(k4[j].x, u, dec * s[4 * j]);
        s[4 * j + 1] = fmaf(k4[j].y, u, dec * s[4 * j + 1]);
        s[4 * j + 2] = fmaf(k4[j].z, u, dec * s[4 * j + 2]);
        s[4 * j + 3] = fmaf(k4[j].w, u, dec * s[4 * j + 3]);
      }
      if (tt + 1 < DR_TILE) {
#pragma unroll
        for (int j = 0; j < ROWS / 4; ++j) {
          k4[j] = k4n[j];
          q4[j] = q4n[j];
        }
        gt = gtn;
      }
    }
    __syncthreads();      // the next round's copies overwrite the buffer that was just read
  }
  pdl_launch_dependents();
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int row = 4 * (LPC * (i >> 2) + sub) + (i & 3);
    if (live && row < dim) S[(size_t)row * vdim + col] = s[i];
  }
}

extern "C" int TL_NAME(tl_delta_prep)(const float* z, int ld, const float* taps_w, int taps, const float* kept,
                                      float* y, int ldy, float* gates, const float* neg_a, const float* dt_bias,
                                      int col_b, int col_a, const int* token_seq, const int* seq_start,
                                      const int* seq_slot, int T, int G, int H, int dim, int vdim, float unit_eps,
                                      float q_scale, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (G < 1 || H < 1 || H % G || dim < 1 || vdim < 1 || taps < 1) return TL_ERR_BAD_ARG;
  if (dim > 32 * DR_MAX_R || taps > DR_MAX_TAPS) return TL_ERR_UNSUPPORTED;
  const int units = G + H;
  int gy = (units + DR_WARPS - 1) / DR_WARPS;
  if (gy > 65535) gy = 65535;
  return tl_launch(delta_prep_kernel, dim3(T, gy), dim3(DR_WARPS * 32), 0, stream, z, ld, taps_w, taps, kept, y,
                   ldy, gates, neg_a, dt_bias, col_b, col_a, token_seq, seq_start, seq_slot, G, H, dim, vdim,
                   unit_eps, q_scale);
}

extern "C" int TL_NAME(tl_conv_state_update)(const float* z, int ld, float* kept, int taps, const int* seq_start,
                                             const int* seq_slot, int B, int channels, cudaStream_t stream) {
  if (B <= 0 || channels <= 0 || taps <= 1) return 0;
  if (taps > DR_MAX_TAPS) return TL_ERR_UNSUPPORTED;
  if (B > 65535) return TL_ERR_UNSUPPORTED;
  return tl_launch(conv_state_update_kernel, dim3((channels + 255) / 256, B), dim3(256), 0, stream, z, ld, kept,
                   taps, seq_start, seq_slot, channels);
}

extern "C" int TL_NAME(tl_delta_scan)(const float* y, int ldy, const float* gates, float* state, float* o, int ldo,
                                      const int* seq_start, const int* seq_slot, int T, int B, int G, int H,
                                      int dim, int vdim, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (G < 1 || H < 1 || H % G || dim < 1 || vdim < 1) return TL_ERR_BAD_ARG;
  const int R = (dim + 31) / 32;
  if (H > 65535 || R > DR_MAX_R) return TL_ERR_UNSUPPORTED;
  if (T >= 8 * B && dim <= 128) {
    // many tokens per sequence: several lanes a column, operands through shared memory
    const int lpc = dim <= 16 ? 4 : (dim <= 32 ? 8 : 16);
    const int cols = 4 * (32 / lpc);
    dim3 tg(B, H, (vdim + cols - 1) / cols);
    if (tg.z > 65535) return TL_ERR_UNSUPPORTED;
#define TILED(ROWS_, LPC_)                                                                                    \
    return tl_launch(delta_scan_tiled_kernel<ROWS_, LPC_>, tg, dim3(128), 0, stream, y, ldy, gates, state, o, \
                     ldo, seq_start, seq_slot, G, H, dim, vdim)
    if (dim <= 16) TILED(4, 4);
    if (dim <= 32) TILED(4, 8);
    if (dim <= 64) TILED(4, 16);
    TILED(8, 16);
#undef TILED
  }
  const int per_block = DR_WARPS * DR_COLS;
  dim3 grid(B, H, (vdim + per_block - 1) / per_block);
  if (grid.z > 65535) return TL_ERR_UNSUPPORTED;
  int rc;
#define SCAN(RR)                                                                                           \
  rc = tl_launch(delta_scan_kernel<RR>, grid, dim3(DR_WARPS * 32), 0, stream, y, ldy, gates, state, o, ldo, \
                 seq_start, seq_slot, G, H, dim, vdim);                                                     \
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

// x[t, c] <- silu(x[t, c]) for the first n columns of 32-bit rows with stride ld.
__global__ void __launch_bounds__(256)
silu_rows_kernel(float* __restrict__ x, int ld, int T, int n) {
  pdl_wait();
  pdl_launch_dependents();
  const long long total = (long long)T * n;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / n), c = (int)(i - (long long)t * n);
    float* p = x + (size_t)t * ld + c;
    *p = dr_silu(*p);
  }
}

__global__ void __launch_bounds__(256)
silu_rows_vec_kernel(float* __restrict__ x, int ld, int T, int n4) {
  pdl_wait();
  pdl_launch_dependents();
  const long long total = (long long)T * n4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / n4), c = (int)(i - (long long)t * n4) * 4;
    float4* p = reinterpret_cast<float4*>(x + (size_t)t * ld + c);
    float4 v = *p;
    v.x = dr_silu(v.x); v.y = dr_silu(v.y); v.z = dr_silu(v.z); v.w = dr_silu(v.w);
    *p = v;
  }
}

extern "C" int TL_NAME(tl_silu_rows)(float* x, int ld, int T, int n, cudaStream_t stream) {
  if (T <= 0 || n <= 0) return 0;
  if (n % 4 == 0 && ld % 4 == 0 && ((uintptr_t)x & 15) == 0) {
    const long long quads = (long long)T * (n / 4);
    const int blocks = (int)((quads + 255) / 256 < 148 * 16 ? (quads + 255) / 256 : 148 * 16);
    return tl_launch(silu_rows_vec_kernel, dim3(blocks), dim3(256), 0, stream, x, ld, T, n / 4);
  }
  const long long total = (long long)T * n;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  return tl_launch(silu_rows_kernel, dim3(blocks), dim3(256), 0, stream, x, ld, T, n);
}

// Mixers side by side, summed with one factor each: out (+)= sum_b scale_b (y_b + bias_b); a bias may be
// absent.  Rows of n 32-bit numbers, contiguous.
#define WS_MAX 4
struct WeightedPtrs {
  const float* y[WS_MAX];
  const float* bias[WS_MAX];
  float scale[WS_MAX];
};

__global__ void __launch_bounds__(256)
weighted_sum_kernel(WeightedPtrs p, int nb, float* __restrict__ out, int T, int n, int accumulate) {
  pdl_wait();
  pdl_launch_dependents();
  const long long total = (long long)T * n;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % n);
    float acc = accumulate ? out[i] : 0.0f;
    for (int b = 0; b < nb; ++b) {
      const float v = p.y[b][i] + (p.bias[b] != nullptr ? p.bias[b][c] : 0.0f);
      acc = fmaf(p.scale[b], v, acc);
    }
    out[i] = acc;
  }
}

extern "C" int TL_NAME(tl_weighted_sum)(const float* const* ys, const float* const* biases, const float* scales,
                                        int nb, float* out, int T, int n, int accumulate, cudaStream_t stream) {
  if (T <= 0 || n <= 0) return 0;
  if (nb < 1 || nb > WS_MAX) return TL_ERR_UNSUPPORTED;
  WeightedPtrs p = {};
  for (int b = 0; b < nb; ++b) {
    p.y[b] = ys[b];
    p.bias[b] = biases[b];
    p.scale[b] = scales[b];
  }
  const long long total = (long long)T * n;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  return tl_launch(weighted_sum_kernel, dim3(blocks), dim3(256), 0, stream, p, nb, out, T, n, accumulate);
}
