// Residual streams kept several at a time (hyper-connections), and the small row kernels of
// mixers that run branches side by side.  Everything here is bound by memory; sums, norms and
// the streams themselves are 32-bit, `act_t` is what feeds the matrix products.
//
// Streams lie token-major: xs[t, s, :] for s < S, so one token's streams are one contiguous run.
// A sublayer reads   u = sum_s a[s] xs[t, s, :]   through a norm, and its output y goes back as
//   xs'[t, j, :] = sum_s M[s, j] xs[t, s, :] + b[j] y[t, :]          (M is indexed [from, to])
// The kernel that writes a sublayer's output can also do the next sublayer's read and norm, so
// the streams cross the memory once per sublayer.
#include "common.cuh"

#define HC_MAX_STREAMS 8

// Threads of a row kernel: one per four coordinates (a row is then one round of 16-byte loads, all in
// flight at once), between 128 and 1024.
static inline int row_threads(int H) {
  int t = ((H + 3) / 4 + 31) / 32 * 32;
  return t < 128 ? 128 : (t > 1024 ? 1024 : t);
}


// xs[t, s, :] = x[t, :] for every s.
__global__ void stream_spread_kernel(const float* __restrict__ x, float* __restrict__ xs, int H, int S) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const float* src = x + (size_t)t * H;
  float* dst = xs + (size_t)t * S * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = src[i];
    for (int s = 0; s < S; ++s) dst[(size_t)s * H + i] = v;
  }
}

extern "C" int TL_NAME(tl_stream_spread)(const float* x, float* xs, int T, int H, int S, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (S < 1 || H < 1) return TL_ERR_BAD_ARG;
  return tl_launch(stream_spread_kernel, dim3(T), dim3(256), 0, stream, x, xs, H, S);
}

// x[r, :] = sum_s xs[rows[r], s, :]   (rows null: row r itself), streams added in their order.
__global__ void stream_sum_kernel(const float* __restrict__ xs, const int* __restrict__ rows,
                                  float* __restrict__ x, int H, int S) {
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const int t = rows != nullptr ? rows[r] : r;
  const float* src = xs + (size_t)t * S * H;
  if ((H & 3) == 0) {
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      float4 a = *reinterpret_cast<const float4*>(src + i);
      for (int s = 1; s < S; ++s) {
        const float4 v = *reinterpret_cast<const float4*>(src + (size_t)s * H + i);
        a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
      }
      *reinterpret_cast<float4*>(x + (size_t)r * H + i) = a;
    }
    return;
  }
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float a = src[i];
    for (int s = 1; s < S; ++s) a += src[(size_t)s * H + i];
    x[(size_t)r * H + i] = a;
  }
}

extern "C" int TL_NAME(tl_stream_sum)(const float* xs, const int* rows, float* x, int R, int H, int S,
                                      cudaStream_t stream) {
  if (R <= 0) return 0;
  if (S < 1 || H < 1) return TL_ERR_BAD_ARG;
  return tl_launch(stream_sum_kernel, dim3(R), dim3(row_threads(H)), 0, stream, xs, rows, x, H, S);
}

// out[t, :] = act( u / sqrt(mean(u^2) + eps) * w ),  u = sum_s a[s] xs[t, s, :].
// `w` is the 32-bit factor per coordinate (a norm whose stored weight lies around zero hands in
// 1 + weight).  u is kept in shared memory between the two passes (H floats).
__global__ void __launch_bounds__(1024)
hc_read_norm_kernel(const float* __restrict__ xs, const float* __restrict__ a, const float* __restrict__ w,
                    float eps, act_t* __restrict__ out, int H, int S) {
  extern __shared__ __align__(16) float u_s[];
  __shared__ float scratch[33];
  __shared__ float a_s[HC_MAX_STREAMS];
  pdl_wait();
  pdl_launch_dependents();
  if (threadIdx.x < S) a_s[threadIdx.x] = a[threadIdx.x];
  __syncthreads();
  const int t = blockIdx.x;
  const float* src = xs + (size_t)t * S * H;
  float ss = 0.0f;
  if ((H & 3) == 0) {
    // 16 bytes per load (rows of the streams start on 16-byte boundaries when H is a multiple of 4)
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      float4 u = *reinterpret_cast<const float4*>(src + i);
      u.x *= a_s[0]; u.y *= a_s[0]; u.z *= a_s[0]; u.w *= a_s[0];
      for (int s = 1; s < S; ++s) {
        const float4 v = *reinterpret_cast<const float4*>(src + (size_t)s * H + i);
        u.x = fmaf(a_s[s], v.x, u.x); u.y = fmaf(a_s[s], v.y, u.y);
        u.z = fmaf(a_s[s], v.z, u.z); u.w = fmaf(a_s[s], v.w, u.w);
      }
      *reinterpret_cast<float4*>(u_s + i) = u;
      ss = fmaf(u.x, u.x, fmaf(u.y, u.y, fmaf(u.z, u.z, fmaf(u.w, u.w, ss))));
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float u = a_s[0] * src[i];
      for (int s = 1; s < S; ++s) u = fmaf(a_s[s], src[(size_t)s * H + i], u);
      u_s[i] = u;
      ss = fmaf(u, u, ss);
    }
  }
  const float total = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(total / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    out[(size_t)t * H + i] = from_f32<act_t>(u_s[i] * inv * w[i]);
}

extern "C" int TL_NAME(tl_hc_read_norm)(const float* xs, const float* a, const float* w, float eps, void* out,
                                        int T, int H, int S, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (S < 1 || S > HC_MAX_STREAMS || H < 1) return TL_ERR_UNSUPPORTED;
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 200 * 1024) return TL_ERR_UNSUPPORTED;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(hc_read_norm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return tl_launch(hc_read_norm_kernel, dim3(T), dim3(row_threads(H)), smem, stream, xs, a, w, eps, (act_t*)out, H, S);
}

// xs'[t, j, :] = sum_s M[s, j] xs[t, s, :] + b[j] y[t, :], in place (a coordinate's S values are
// read before any is written).  With `a2` given the kernel goes on to the next sublayer's read:
// out2[t, :] = act( u2 / rms(u2) * w2 ) with u2 = sum_j a2[j] xs'[t, j, :].
__global__ void __launch_bounds__(1024)
hc_write_kernel(float* __restrict__ xs, const float* __restrict__ M, const float* __restrict__ b,
                const float* __restrict__ y, int ldy, int H, int S, const float* __restrict__ a2,
                const float* __restrict__ w2, float eps2, act_t* __restrict__ out2) {
  extern __shared__ __align__(16) float u_s[];
  __shared__ float scratch[33];
  __shared__ float m_s[HC_MAX_STREAMS * HC_MAX_STREAMS], b_s[HC_MAX_STREAMS], a_s[HC_MAX_STREAMS];
  pdl_wait();
  pdl_launch_dependents();
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) m_s[i] = M[i];
  if (threadIdx.x < S) {
    b_s[threadIdx.x] = b[threadIdx.x];
    a_s[threadIdx.x] = a2 != nullptr ? a2[threadIdx.x] : 0.0f;
  }
  __syncthreads();
  const int t = blockIdx.x;
  float* row = xs + (size_t)t * S * H;
  const float* yr = y + (size_t)t * ldy;
  float ss = 0.0f;
  if ((H & 3) == 0 && (ldy & 3) == 0 && S <= 4) {
    // four coordinates per thread, 16 bytes per load and store (the usual case of up to four streams)
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      float4 old[4];
#pragma unroll
      for (int s = 0; s < 4; ++s)
        old[s] = s < S ? *reinterpret_cast<const float4*>(row + (size_t)s * H + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      const float4 yv = *reinterpret_cast<const float4*>(yr + i);
      float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (j < S) {
          float4 v;
          v.x = m_s[j] * old[0].x; v.y = m_s[j] * old[0].y; v.z = m_s[j] * old[0].z; v.w = m_s[j] * old[0].w;
#pragma unroll
          for (int s = 1; s < 4; ++s)
            if (s < S) {
              const float m = m_s[s * S + j];
              v.x = fmaf(m, old[s].x, v.x); v.y = fmaf(m, old[s].y, v.y);
              v.z = fmaf(m, old[s].z, v.z); v.w = fmaf(m, old[s].w, v.w);
            }
          v.x = fmaf(b_s[j], yv.x, v.x); v.y = fmaf(b_s[j], yv.y, v.y);
          v.z = fmaf(b_s[j], yv.z, v.z); v.w = fmaf(b_s[j], yv.w, v.w);
          *reinterpret_cast<float4*>(row + (size_t)j * H + i) = v;
          if (j == 0) { u.x = a_s[0] * v.x; u.y = a_s[0] * v.y; u.z = a_s[0] * v.z; u.w = a_s[0] * v.w; }
          else {
            u.x = fmaf(a_s[j], v.x, u.x); u.y = fmaf(a_s[j], v.y, u.y);
            u.z = fmaf(a_s[j], v.z, u.z); u.w = fmaf(a_s[j], v.w, u.w);
          }
        }
      }
      if (a2 != nullptr) {
        *reinterpret_cast<float4*>(u_s + i) = u;
        ss = fmaf(u.x, u.x, fmaf(u.y, u.y, fmaf(u.z, u.z, fmaf(u.w, u.w, ss))));
      }
    }
  } else
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float old[HC_MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < HC_MAX_STREAMS; ++s) old[s] = s < S ? row[(size_t)s * H + i] : 0.0f;
    const float yv = yr[i];
    float u = 0.0f;
#pragma unroll
    for (int j = 0; j < HC_MAX_STREAMS; ++j) {
      if (j < S) {
        float v = m_s[j] * old[0];
#pragma unroll
        for (int s = 1; s < HC_MAX_STREAMS; ++s)
          if (s < S) v = fmaf(m_s[s * S + j], old[s], v);
        v = fmaf(b_s[j], yv, v);
        row[(size_t)j * H + i] = v;
        u = j == 0 ? a_s[0] * v : fmaf(a_s[j], v, u);
      }
    }
    if (a2 != nullptr) {
      u_s[i] = u;
      ss = fmaf(u, u, ss);
    }
  }
  if (a2 == nullptr) return;
  const float total = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(total / (float)H + eps2);
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    out2[(size_t)t * H + i] = from_f32<act_t>(u_s[i] * inv * w2[i]);
}

extern "C" int TL_NAME(tl_hc_write)(float* xs, const float* M, const float* b, const float* y, int ldy, int T,
                                    int H, int S, const float* a2, const float* w2, float eps2, void* out2,
                                    cudaStream_t stream) {
  if (T <= 0) return 0;
  if (S < 1 || S > HC_MAX_STREAMS || H < 1) return TL_ERR_UNSUPPORTED;
  if (a2 != nullptr && (w2 == nullptr || out2 == nullptr)) return TL_ERR_BAD_ARG;
  const size_t smem = a2 != nullptr ? (size_t)H * sizeof(float) : 0;
  if (smem > 200 * 1024) return TL_ERR_UNSUPPORTED;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(hc_write_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return tl_launch(hc_write_kernel, dim3(T), dim3(row_threads(H)), smem, stream, xs, M, b, y, ldy, H, S, a2, w2, eps2,
                   (act_t*)out2);
}

// Branches side by side: out[t, :] (+)= (1 / n) sum_b y_b[t, :] / sqrt(mean(y_b[t]^2) + eps) * w_b[:],
// each branch's output normalised over the whole row with its own 32-bit weight.
#define BR_MAX 4
struct BranchPtrs {
  const float* y[BR_MAX];
  const float* w[BR_MAX];
};

__global__ void __launch_bounds__(1024)
branch_norm_mean_kernel(BranchPtrs p, int n, int H, float eps, float* __restrict__ out, int accumulate) {
  __shared__ float scratch[33];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  float inv[BR_MAX];
  const bool vec = (H & 3) == 0;
  const float share0 = 1.0f / (float)n;
  if (vec && H <= 4 * (int)blockDim.x) {
    // a row is one round of loads: every branch's four values stay in registers between the sum of
    // squares and the scaling, so the outputs are read once
    const int i = threadIdx.x * 4;
    float4 v[BR_MAX];
#pragma unroll
    for (int b = 0; b < BR_MAX; ++b) {
      v[b] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (b < n && i < H) v[b] = *reinterpret_cast<const float4*>(p.y[b] + (size_t)t * H + i);
    }
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int b = 0; b < BR_MAX; ++b) {
      if (b < n) {
        const float ss = fmaf(v[b].x, v[b].x, fmaf(v[b].y, v[b].y, fmaf(v[b].z, v[b].z, v[b].w * v[b].w)));
        const float total = block_sum(ss, scratch);
        const float r = 1.0f / sqrtf(total / (float)H + eps);
        if (i < H) {
          const float4 w = *reinterpret_cast<const float4*>(p.w[b] + i);
          a.x += v[b].x * r * w.x; a.y += v[b].y * r * w.y; a.z += v[b].z * r * w.z; a.w += v[b].w * r * w.w;
        }
      }
    }
    if (i < H) {
      a.x *= share0; a.y *= share0; a.z *= share0; a.w *= share0;
      float4* o = reinterpret_cast<float4*>(out + (size_t)t * H + i);
      if (accumulate) { const float4 c = *o; a.x += c.x; a.y += c.y; a.z += c.z; a.w += c.w; }
      *o = a;
    }
    return;
  }
  for (int b = 0; b < n; ++b) {
    const float* y = p.y[b] + (size_t)t * H;
    float ss = 0.0f;
    if (vec) {
      for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4*>(y + i);
        ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
      }
    } else {
      for (int i = threadIdx.x; i < H; i += blockDim.x) ss = fmaf(y[i], y[i], ss);
    }
    const float total = block_sum(ss, scratch);
    inv[b] = 1.0f / sqrtf(total / (float)H + eps);
  }
  const float share = 1.0f / (float)n;
  if (vec) {
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int b = 0; b < n; ++b) {
        const float4 v = *reinterpret_cast<const float4*>(p.y[b] + (size_t)t * H + i);
        const float4 w = *reinterpret_cast<const float4*>(p.w[b] + i);
        a.x += v.x * inv[b] * w.x; a.y += v.y * inv[b] * w.y; a.z += v.z * inv[b] * w.z; a.w += v.w * inv[b] * w.w;
      }
      a.x *= share; a.y *= share; a.z *= share; a.w *= share;
      float4* o = reinterpret_cast<float4*>(out + (size_t)t * H + i);
      if (accumulate) { const float4 c = *o; a.x += c.x; a.y += c.y; a.z += c.z; a.w += c.w; }
      *o = a;
    }
    return;
  }
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float a = 0.0f;
    for (int b = 0; b < n; ++b) a += p.y[b][(size_t)t * H + i] * inv[b] * p.w[b][i];
    a *= share;
    float* o = out + (size_t)t * H + i;
    *o = accumulate ? *o + a : a;
  }
}

extern "C" int TL_NAME(tl_branch_norm_mean)(const float* const* ys, const float* const* ws, int n, int T, int H,
                                            float eps, float* out, int accumulate, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n < 1 || n > BR_MAX) return TL_ERR_UNSUPPORTED;
  BranchPtrs p = {};
  for (int b = 0; b < n; ++b) {
    p.y[b] = ys[b];
    p.w[b] = ws[b];
  }
  return tl_launch(branch_norm_mean_kernel, dim3(T), dim3(row_threads(H)), 0, stream, p, n, H, eps, out, accumulate);
}

// Per-head output norm with a gate: out[t, h, :] = act( o[t, h, :] / rms * w[:] * f(g[t, h, :]) ),
// the norm over the head's `vdim` entries with one weight vector for all heads; f is silu (gate_act 0)
// or the sigmoid (1).  A warp per (t, h).  (One "head" of the row's whole width is a norm over the
// concatenated heads.)
__global__ void __launch_bounds__(256)
headnorm_silu_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, float eps,
                          const float* __restrict__ g, int ldg, act_t* __restrict__ out, int rows, int heads,
                          int vdim, int gate_act) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int t = r / heads, h = r - t * heads;
  const float* src = o + (size_t)r * vdim;
  const float* gate = g + (size_t)t * ldg + (size_t)h * vdim;
  float ss = 0.0f;
  for (int i = lane; i < vdim; i += 32) ss = fmaf(src[i], src[i], ss);
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
  for (int i = lane; i < vdim; i += 32) {
    const float z = gate[i];
    const float sg = 1.0f / (1.0f + expf(-z));
    out[(size_t)r * vdim + i] = from_f32<act_t>(src[i] * inv * w[i] * (gate_act == 0 ? z * sg : sg));
  }
}

// The same for heads too wide for a warp (a norm over the concatenated heads of a whole row): a block per
// (t, h), the sum of squares over the block, the row read a second time from cache.  Few rows (decode
// steps) get blocks of 1024 threads, so that a thread's loads are few and in flight together.
__global__ void __launch_bounds__(1024)
headnorm_gate_wide_kernel(const float* __restrict__ o, const float* __restrict__ w, float eps,
                          const float* __restrict__ g, int ldg, act_t* __restrict__ out, int heads, int vdim,
                          int gate_act) {
  __shared__ float scratch[33];
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const int t = r / heads, h = r - t * heads;
  const float* src = o + (size_t)r * vdim;
  const float* gate = g + (size_t)t * ldg + (size_t)h * vdim;
  float ss = 0.0f;
#pragma unroll 4
  for (int i = threadIdx.x; i < vdim; i += blockDim.x) ss = fmaf(src[i], src[i], ss);
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
  for (int i = threadIdx.x; i < vdim; i += blockDim.x) {
    const float z = gate[i];
    const float sg = 1.0f / (1.0f + expf(-z));
    out[(size_t)r * vdim + i] = from_f32<act_t>(src[i] * inv * w[i] * (gate_act == 0 ? z * sg : sg));
  }
}

extern "C" int TL_NAME(tl_headnorm_silu_gate)(const float* o, const float* w, float eps, const float* g, int ldg,
                                              void* out, int T, int heads, int vdim, int gate_act,
                                              cudaStream_t stream) {
  if (T <= 0) return 0;
  if (heads < 1 || vdim < 1) return TL_ERR_BAD_ARG;
  const long long rows = (long long)T * heads;
  if (rows > 0x7fffffffLL) return TL_ERR_UNSUPPORTED;
  if (vdim > 512)
    return tl_launch(headnorm_gate_wide_kernel, dim3((unsigned)rows), dim3(vdim >= 2048 && rows < 512 ? 1024 : 256), 0, stream, o, w, eps, g, ldg,
                     (act_t*)out, heads, vdim, gate_act);
  const unsigned blocks = (unsigned)((rows + 7) / 8);
  return tl_launch(headnorm_silu_gate_kernel, dim3(blocks), dim3(256), 0, stream, o, w, eps, g, ldg, (act_t*)out,
                   (int)rows, heads, vdim, gate_act);
}
