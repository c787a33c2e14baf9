// Mixture of experts: router, the grouping of (token, expert) pairs by expert, the experts'
// products over each group, and the weighted sum per token.
//
//   scores s = softmax(z) over all router outputs (32-bit); the choice is made on s + correction,
//   the `top` largest (ties: the lower index); the weights are the chosen s, not renormalised.
//   Router outputs from `experts` on have no matrices: such an expert hands its input through.
//   A real expert: g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit),
//                  y = W_down( g * sigmoid(alpha g) * (u + 1) ).
//
// Nothing here needs the host: counts and offsets stay on the device, and the product kernels are
// launched over an upper bound of tiles, of which a block finds its own (expert, rows) or leaves.
// A token's result is the sum of its chosen experts' outputs in the order of its choice, so it does
// not depend on what else is in the step.
#include "common.cuh"

#define MOE_MAX_PER_LANE 16     // router outputs per lane: up to 512 experts

__global__ void __launch_bounds__(256)
moe_route_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ corr, int n_out, int top,
                 int* __restrict__ idx, float* __restrict__ wt, int T) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const float* row = z + (size_t)t * ldz;
  float s[MOE_MAX_PER_LANE], c[MOE_MAX_PER_LANE];
  float m = -INFINITY;
#pragma unroll
  for (int r = 0; r < MOE_MAX_PER_LANE; ++r) {
    const int e = lane + 32 * r;
    s[r] = e < n_out ? row[e] : -INFINITY;
    m = fmaxf(m, s[r]);
  }
  m = warp_max(m);
  float sum = 0.0f;
#pragma unroll
  for (int r = 0; r < MOE_MAX_PER_LANE; ++r) {
    s[r] = lane + 32 * r < n_out ? expf(s[r] - m) : 0.0f;
    sum += s[r];
  }
  sum = warp_sum(sum);
#pragma unroll
  for (int r = 0; r < MOE_MAX_PER_LANE; ++r) {
    const int e = lane + 32 * r;
    s[r] = s[r] / sum;
    c[r] = e < n_out ? s[r] + (corr != nullptr ? corr[e] : 0.0f) : -INFINITY;
  }
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY, best_s = 0.0f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int r = 0; r < MOE_MAX_PER_LANE; ++r) {
      const int e = lane + 32 * r;
      if (e < n_out && c[r] > best) {    // r rises with e, so a tie keeps the lower index
        best = c[r];
        best_e = e;
        best_s = s[r];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      const float os = __shfl_xor_sync(0xffffffffu, best_s, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
        best_s = os;
      }
    }
    if (lane == 0) {
      idx[(size_t)t * top + k] = best_e;
      wt[(size_t)t * top + k] = best_s;
    }
#pragma unroll
    for (int r = 0; r < MOE_MAX_PER_LANE; ++r)
      if (lane + 32 * r == best_e) c[r] = -INFINITY;
  }
}

extern "C" int TL_NAME(tl_moe_route)(const float* z, int ldz, const float* corr, int n_out, int top, int* idx,
                                     float* wt, int T, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n_out < 1 || top < 1 || top > n_out) return TL_ERR_BAD_ARG;
  if (n_out > 32 * MOE_MAX_PER_LANE) return TL_ERR_UNSUPPORTED;
  return tl_launch(moe_route_kernel, dim3((T + 7) / 8), dim3(256), 0, stream, z, ldz, corr, n_out, top, idx, wt,
                   T);
}

// The choice among grouped experts by sigmoid scores.
//   s = sigmoid(z) (32-bit).  The n_out experts form `groups` equal groups of neighbours; a group's
//   score is the sum of its two largest s (of its one, if groups have one member); only experts of
//   the `keep` best groups can be chosen (ties: the lower group); among them the `top` largest s are
//   chosen (ties: the lower index); their weights are s / (sum of the chosen s + 1e-20) * scale.
// A warp per token; scores, group scores and group flags in the warp's shared memory.
#define MOE_GROUPED_WARPS 4
#define MOE_GROUPED_MAX 512
__global__ void __launch_bounds__(MOE_GROUPED_WARPS * 32)
moe_route_grouped_kernel(const float* __restrict__ z, int ldz, int n_out, int groups, int keep, int top,
                         float scale, int* __restrict__ idx, float* __restrict__ wt, int T) {
  __shared__ float sc[MOE_GROUPED_WARPS][MOE_GROUPED_MAX];
  __shared__ float gs[MOE_GROUPED_WARPS][MOE_GROUPED_MAX];
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * MOE_GROUPED_WARPS + warp;
  if (t >= T) return;
  const float* row = z + (size_t)t * ldz;
  float* s = sc[warp];
  float* g = gs[warp];
  const int size = n_out / groups;
  for (int e = lane; e < n_out; e += 32) s[e] = 1.0f / (1.0f + expf(-row[e]));
  __syncwarp();
  for (int k = lane; k < groups; k += 32) {
    float a = -INFINITY, b = -INFINITY;     // the largest and the second
    for (int e = k * size; e < (k + 1) * size; ++e) {
      const float v = s[e];
      if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
    }
    g[k] = size > 1 ? a + b : a;
  }
  __syncwarp();
  // the `keep` best groups stay; the others' scores are struck out
  if (keep < groups) {
    for (int round = 0; round < keep; ++round) {
      float best = -INFINITY;
      int best_k = 0x7fffffff;
      for (int k = lane; k < groups; k += 32)
        if (g[k] != INFINITY && g[k] > best) { best = g[k]; best_k = k; }   // k rises: a tie keeps the lower group
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int ok = __shfl_xor_sync(0xffffffffu, best_k, o);
        if (ob > best || (ob == best && ok < best_k)) { best = ob; best_k = ok; }
      }
      if (lane == 0 && best_k < groups) g[best_k] = INFINITY;     // marks a kept group
      __syncwarp();
    }
    for (int e = lane; e < n_out; e += 32)
      if (g[e / size] != INFINITY) s[e] = -1.0f;                  // below every sigmoid
    __syncwarp();
  }
  float sum = 0.0f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int e = lane; e < n_out; e += 32)
      if (s[e] > best) { best = s[e]; best_e = e; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    if (lane == 0) {
      idx[(size_t)t * top + k] = best_e;
      wt[(size_t)t * top + k] = best;
      s[best_e] = -2.0f;
    }
    sum += best;
    __syncwarp();
  }
  const float f = scale / (sum + 1e-20f);
  for (int k = lane; k < top; k += 32) wt[(size_t)t * top + k] *= f;
}

extern "C" int TL_NAME(tl_moe_route_grouped)(const float* z, int ldz, int n_out, int groups, int keep, int top,
                                             float scale, int* idx, float* wt, int T, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n_out < 1 || groups < 1 || n_out % groups || keep < 1 || keep > groups || top < 1 ||
      top > keep * (n_out / groups))
    return TL_ERR_BAD_ARG;
  if (n_out > MOE_GROUPED_MAX) return TL_ERR_UNSUPPORTED;
  return tl_launch(moe_route_grouped_kernel, dim3((T + MOE_GROUPED_WARPS - 1) / MOE_GROUPED_WARPS),
                   dim3(MOE_GROUPED_WARPS * 32), 0, stream, z, ldz, n_out, groups, keep, top, scale, idx, wt, T);
}

// Groups the pairs by expert.  offsets[e] .. offsets[e + 1] are the rows of expert e < E in the
// grouped order; row_token[row] is the token a row belongs to; row_of[pair] is the row of pair
// (t, k), or -1 for a pair whose expert hands its input through.  One block: the pairs of a step
// are few against what the products move.
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ idx, int n_pairs, int top, int E, int* __restrict__ offsets,
                int* __restrict__ row_token, int* __restrict__ row_of) {
  extern __shared__ int sm[];
  int* count = sm;            // [E]
  int* start = sm + E;        // [E + 1]
  pdl_wait();
  pdl_launch_dependents();
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = idx[p];
    if (e < E) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = at;
      at += count[e];
    }
    start[E] = at;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) {
    offsets[e] = start[e];
    if (e < E) count[e] = 0;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = idx[p];
    if (e < E) {
      const int row = start[e] + atomicAdd(&count[e], 1);
      row_token[row] = p / top;
      row_of[p] = row;
    } else {
      row_of[p] = -1;
    }
  }
}

extern "C" int TL_NAME(tl_moe_plan)(const int* idx, int n_pairs, int top, int E, int* offsets, int* row_token,
                                    int* row_of, cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  if (E < 0 || E > 4096 || top < 1) return TL_ERR_UNSUPPORTED;
  return tl_launch(moe_plan_kernel, dim3(1), dim3(1024), (size_t)(2 * E + 1) * sizeof(int), stream, idx, n_pairs,
                   top, E, offsets, row_token, row_of);
}

// ---------------------------------------------------------------------------
// The experts' products over the grouped rows, on CUDA cores with 32-bit accumulation:
//   UP:    C[row, n] (act_t) = act( A[row_token[row]] . Wg_e[n], A[row_token[row]] . Wu_e[n] )
//          with W_e = [2 N, K]: N gate rows, then N up rows
//   DOWN:  C[row, n] (float) = A[row] . W_e[n],  W_e = [N, K]
// Block y walks an upper bound of row tiles (pairs / 64 + experts); it finds the expert whose
// rows its tile covers from the offsets, or leaves.
// ---------------------------------------------------------------------------
#define GBM 64
#define GBN 64
#define GBK 16

template <bool UP>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const act_t* __restrict__ A, int lda, const int* __restrict__ row_token,
                const act_t* __restrict__ W, void* __restrict__ C, int ldc, const int* __restrict__ offsets,
                int E, int N, int K, float limit, float alpha) {
  __shared__ float As[GBK][GBM + 4];
  __shared__ float Ws[GBK][GBN + 4];
  __shared__ float Us[UP ? GBK : 1][GBN + 4];
  __shared__ int src_row[GBM];
  __shared__ int tile_info[3];   // expert, first row, rows
  pdl_wait();
  const int tid = threadIdx.x;
  if (tid == 0) {
    int tile = blockIdx.y, e = 0, found = -1;
    for (; e < E; ++e) {
      const int cnt = offsets[e + 1] - offsets[e];
      const int tiles = (cnt + GBM - 1) / GBM;
      if (tile < tiles) {
        found = e;
        break;
      }
      tile -= tiles;
    }
    tile_info[0] = found;
    if (found >= 0) {
      tile_info[1] = offsets[found] + tile * GBM;
      const int left = offsets[found + 1] - tile_info[1];
      tile_info[2] = left < GBM ? left : GBM;
    }
  }
  __syncthreads();
  const int e = tile_info[0];
  if (e < 0) return;
  const int r0 = tile_info[1], rows = tile_info[2];
  if (tid < GBM) src_row[tid] = tid < rows ? (UP ? row_token[r0 + tid] : r0 + tid) : -1;
  __syncthreads();
  const act_t* We = W + (size_t)e * (UP ? 2 : 1) * N * K;
  const int tx = tid & 15, ty = tid >> 4;
  const int n0 = blockIdx.x * GBN;
  float acc[4][4] = {}, acu[4][4] = {};
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  const int arow = src_row[lrow];
  for (int k0 = 0; k0 < K; k0 += GBK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lk + j;
      const int wn = n0 + lrow;
      As[lk + j][lrow] = (arow >= 0 && k < K) ? to_f32(A[(size_t)arow * lda + k]) : 0.0f;
      Ws[lk + j][lrow] = (wn < N && k < K) ? to_f32(We[(size_t)wn * K + k]) : 0.0f;
      if (UP) Us[lk + j][lrow] = (wn < N && k < K) ? to_f32(We[(size_t)(N + wn) * K + k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < GBK; ++k) {
      float a[4], w[4], u[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
      if (UP) {
#pragma unroll
        for (int j = 0; j < 4; ++j) u[j] = Us[k][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
          if (UP) acu[i][j] = fmaf(a[i], u[j], acu[i][j]);
        }
    }
    __syncthreads();
  }
  pdl_launch_dependents();   // only now: a grid let go earlier would sit on the SMs and take issue slots
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = ty * 4 + i;
    if (m >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      if (UP) {
        const float g = fminf(acc[i][j], limit);
        const float u = fminf(fmaxf(acu[i][j], -limit), limit);
        ((act_t*)C)[(size_t)(r0 + m) * ldc + n] = from_f32<act_t>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
      } else {
        ((float*)C)[(size_t)(r0 + m) * ldc + n] = acc[i][j];
      }
    }
  }
}

extern "C" int TL_NAME(tl_moe_gemm)(const void* A, int lda, const int* row_token, const void* W, void* C, int ldc,
                                    const int* offsets, int E, int max_rows, int N, int K, int up, float limit,
                                    float alpha, cudaStream_t stream) {
  if (max_rows <= 0 || E <= 0) return 0;
  if (N < 1 || K < 1) return TL_ERR_BAD_ARG;
  const int tiles = (max_rows + GBM - 1) / GBM + E;
  if (tiles > 65535) return TL_ERR_UNSUPPORTED;
  dim3 grid((N + GBN - 1) / GBN, tiles);
  if (up)
    return tl_launch(moe_gemm_kernel<true>, grid, dim3(256), 0, stream, (const act_t*)A, lda, row_token,
                     (const act_t*)W, C, ldc, offsets, E, N, K, limit, alpha);
  return tl_launch(moe_gemm_kernel<false>, grid, dim3(256), 0, stream, (const act_t*)A, lda, row_token,
                   (const act_t*)W, C, ldc, offsets, E, N, K, limit, alpha);
}

// out[t, :] (+)= sum_k wt[t, k] * ( row_of[t, k] >= 0 ? yk[row_of[t, k], :] : h[t, :] ), k in order.
__global__ void __launch_bounds__(1024)
moe_combine_kernel(const float* __restrict__ yk, const int* __restrict__ row_of, const float* __restrict__ wt,
                   const act_t* __restrict__ h, float* __restrict__ out, int ldo, int H, int top, int accumulate) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  if ((H & 3) == 0 && (ldo & 3) == 0) {
    // four coordinates per thread: a token's rows are one round of 16-byte loads
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int k = 0; k < top; ++k) {
        const int row = row_of[(size_t)t * top + k];
        const float w = wt[(size_t)t * top + k];
        float4 v;
        if (row >= 0) {
          v = *reinterpret_cast<const float4*>(yk + (size_t)row * H + i);
        } else {
          const act_t* hp = h + (size_t)t * H + i;
          v = make_float4(to_f32(hp[0]), to_f32(hp[1]), to_f32(hp[2]), to_f32(hp[3]));
        }
        a.x = fmaf(w, v.x, a.x); a.y = fmaf(w, v.y, a.y); a.z = fmaf(w, v.z, a.z); a.w = fmaf(w, v.w, a.w);
      }
      float4* o = reinterpret_cast<float4*>(out + (size_t)t * ldo + i);
      if (accumulate) { const float4 c = *o; a.x += c.x; a.y += c.y; a.z += c.z; a.w += c.w; }
      *o = a;
    }
    return;
  }
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float a = 0.0f;
    for (int k = 0; k < top; ++k) {
      const int row = row_of[(size_t)t * top + k];
      const float v = row >= 0 ? yk[(size_t)row * H + i] : to_f32(h[(size_t)t * H + i]);
      a = fmaf(wt[(size_t)t * top + k], v, a);
    }
    float* o = out + (size_t)t * ldo + i;
    *o = accumulate ? *o + a : a;
  }
}

extern "C" int TL_NAME(tl_moe_combine)(const float* yk, const int* row_of, const float* wt, const void* h,
                                       float* out, int ldo, int T, int H, int top, int accumulate,
                                       cudaStream_t stream) {
  if (T <= 0) return 0;
  int threads = ((H + 3) / 4 + 31) / 32 * 32;
  threads = threads < 128 ? 128 : (threads > 1024 ? 1024 : threads);
  return tl_launch(moe_combine_kernel, dim3(T), dim3(threads), 0, stream, yk, row_of, wt, (const act_t*)h, out, ldo,
                   H, top, accumulate);
}

#if TL_DTYPE == 1
// ---------------------------------------------------------------------------
// The same grouped products on tensor cores (bfloat16): a block takes 64 rows of one expert's group
// and 64 output columns (the gate and the up columns of the same numbers together); operands come in
// steps of 32 along K through shared memory with cp.async, three steps in flight; mma.sync m16n8k16
// with fragments by ldmatrix from swizzled tiles, a warp per 16 rows.  A weight matrix [N][K] is the
// B operand as it lies.  With few rows per expert (decode) the blocks mostly stream weights, which is
// then the whole cost.
// ---------------------------------------------------------------------------
#define MBM 64
#define MBN 64
#define MBK 32
#define MSTAGES 3
typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void moe_cp_async16(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void moe_ldmatrix_x4(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void moe_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// rows of 32 elements are four 16-byte chunks; chunk c of row r lies at c ^ ((r >> 1) & 3)
__device__ __forceinline__ int moe_swz(int row, int chunk) { return chunk ^ ((row >> 1) & 3); }

template <bool UP>
__global__ void __launch_bounds__(128)
moe_gemm_mma_kernel(const bf16* __restrict__ A, int lda, const int* __restrict__ row_token,
                    const bf16* __restrict__ W, void* __restrict__ C, int ldc, const int* __restrict__ offsets,
                    int E, int N, int K, float limit, float alpha) {
  __shared__ __align__(128) bf16 As[MSTAGES][MBM * MBK];
  __shared__ __align__(128) bf16 Ws[MSTAGES][MBN * MBK];
  __shared__ __align__(128) bf16 Us[UP ? MSTAGES : 1][UP ? MBN * MBK : 8];
  __shared__ int src_row[MBM];
  __shared__ int tile_info[3];
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
    int tile = blockIdx.y, e = 0, found = -1;
    for (; e < E; ++e) {
      const int tiles = (offsets[e + 1] - offsets[e] + MBM - 1) / MBM;
      if (tile < tiles) { found = e; break; }
      tile -= tiles;
    }
    tile_info[0] = found;
    if (found >= 0) {
      tile_info[1] = offsets[found] + tile * MBM;
      const int left = offsets[found + 1] - tile_info[1];
      tile_info[2] = left < MBM ? left : MBM;
    }
  }
  __syncthreads();
  const int e = tile_info[0];
  if (e < 0) return;
  const int r0 = tile_info[1], rows = tile_info[2];
  if (tid < MBM) src_row[tid] = tid < rows ? (UP ? row_token[r0 + tid] : r0 + tid) : -1;
  __syncthreads();
  const bf16* We = W + (size_t)e * (UP ? 2 : 1) * N * K;
  const int n0 = blockIdx.x * MBN;
  const int k_iters = (K + MBK - 1) / MBK;

  auto load_stage = [&](int ki, int st) {
    const int k0 = ki * MBK;
    // 64 rows x 4 chunks per operand: two chunks per thread and operand
    for (int i = tid; i < MBM * 4; i += 128) {
      const int row = i >> 2, chunk = i & 3;
      const int k = k0 + chunk * 8;
      bf16* da = &As[st][row * MBK + moe_swz(row, chunk) * 8];
      const int ar = src_row[row];
      if (ar >= 0 && k < K) moe_cp_async16(da, A + (size_t)ar * lda + k);
      else *reinterpret_cast<uint4*>(da) = make_uint4(0, 0, 0, 0);
      bf16* dw = &Ws[st][row * MBK + moe_swz(row, chunk) * 8];
      const int wn = n0 + row;
      if (wn < N && k < K) moe_cp_async16(dw, We + (size_t)wn * K + k);
      else *reinterpret_cast<uint4*>(dw) = make_uint4(0, 0, 0, 0);
      if (UP) {
        bf16* du = &Us[st][row * MBK + moe_swz(row, chunk) * 8];
        if (wn < N && k < K) moe_cp_async16(du, We + (size_t)(N + wn) * K + k);
        else *reinterpret_cast<uint4*>(du) = make_uint4(0, 0, 0, 0);
      }
    }
  };
  float acc[MBN / 8][4], acu[UP ? MBN / 8 : 1][4];
#pragma unroll
  for (int n = 0; n < MBN / 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;
  if (UP) {
#pragma unroll
    for (int n = 0; n < MBN / 8; ++n) acu[n][0] = acu[n][1] = acu[n][2] = acu[n][3] = 0.0f;
  }
#pragma unroll
  for (int s = 0; s < MSTAGES - 1; ++s) {
    if (s < k_iters) load_stage(s, s);
    asm volatile("cp.async.commit_group;");
  }
  for (int ki = 0; ki < k_iters; ++ki) {
    const int st = ki % MSTAGES;
    asm volatile("cp.async.wait_group %0;" ::"n"(MSTAGES - 2));
    __syncthreads();                                     // stage ki is there, and stage ki - 1 is free
    if (ki + MSTAGES - 1 < k_iters) load_stage(ki + MSTAGES - 1, (ki + MSTAGES - 1) % MSTAGES);
    asm volatile("cp.async.commit_group;");
#pragma unroll
    for (int kk = 0; kk < MBK / 16; ++kk) {
      unsigned af[4];
      {
        const int row = warp * 16 + (lane & 15), chunk = kk * 2 + (lane >> 4);
        moe_ldmatrix_x4(af, &As[st][row * MBK + moe_swz(row, chunk) * 8]);
      }
#pragma unroll
      for (int np = 0; np < MBN / 16; ++np) {
        const int row = np * 16 + (lane >> 4) * 8 + (lane & 7), chunk = kk * 2 + ((lane >> 3) & 1);
        unsigned bfr[4];
        moe_ldmatrix_x4(bfr, &Ws[st][row * MBK + moe_swz(row, chunk) * 8]);
        moe_mma(acc[2 * np], af, bfr[0], bfr[1]);
        moe_mma(acc[2 * np + 1], af, bfr[2], bfr[3]);
        if (UP) {
          moe_ldmatrix_x4(bfr, &Us[st][row * MBK + moe_swz(row, chunk) * 8]);
          moe_mma(acu[2 * np], af, bfr[0], bfr[1]);
          moe_mma(acu[2 * np + 1], af, bfr[2], bfr[3]);
        }
      }
    }
  }
  pdl_launch_dependents();   // only now: a grid let go earlier would sit on the SMs and take issue slots
  asm volatile("cp.async.wait_group 0;");
  const int ra = warp * 16 + (lane >> 2), rb = ra + 8;
#pragma unroll
  for (int n = 0; n < MBN / 8; ++n) {
    const int c = n0 + n * 8 + (lane & 3) * 2;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int m = half ? rb : ra;
      if (m >= rows) continue;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        if (c + j >= N) continue;
        const float v = acc[n][half * 2 + j];
        if (UP) {
          const float g = fminf(v, limit);
          const float u = fminf(fmaxf(acu[n][half * 2 + j], -limit), limit);
          ((bf16*)C)[(size_t)(r0 + m) * ldc + c + j] = __float2bfloat16_rn(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
        } else {
          ((float*)C)[(size_t)(r0 + m) * ldc + c + j] = v;
        }
      }
    }
  }
}

extern "C" int tl_moe_gemm_mma(const void* A, int lda, const int* row_token, const void* W, void* C, int ldc,
                               const int* offsets, int E, int max_rows, int N, int K, int up, float limit,
                               float alpha, cudaStream_t stream) {
  if (max_rows <= 0 || E <= 0) return 0;
  if (N < 1 || K < 1) return TL_ERR_BAD_ARG;
  if (K % 8 || lda % 8 || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return TL_ERR_UNSUPPORTED;
  const int tiles = (max_rows + MBM - 1) / MBM + E;
  if (tiles > 65535) return TL_ERR_UNSUPPORTED;
  dim3 grid((N + MBN - 1) / MBN, tiles);
  if (up)
    return tl_launch(moe_gemm_mma_kernel<true>, grid, dim3(128), 0, stream, (const bf16*)A, lda, row_token,
                     (const bf16*)W, C, ldc, offsets, E, N, K, limit, alpha);
  return tl_launch(moe_gemm_mma_kernel<false>, grid, dim3(128), 0, stream, (const bf16*)A, lda, row_token,
                   (const bf16*)W, C, ldc, offsets, E, N, K, limit, alpha);
}
#endif
