// Attention through low-rank latents over a paged cache of one vector per position.
//
// A position's cached vector is [c (rank numbers, normalised) | r (rot numbers, rotated)]: the
// compressed keys/values and the rotated key part that all heads share.  A head's key is W_uk c
// and its value W_uv c, but neither is ever formed: the query's unrotated part is carried into
// the latent space once (qa = W_uk^T q), scores are (qa . c + q_rot . r) * scale, the weighted
// sum of the c's is taken, and W_uv is applied to that sum.  Per position and head the work is
// then that of one key head of width rank + rot shared by all query heads, and the cache holds
// rank + rot numbers per position whatever the number of heads.
//
// Three kernels: what is written per token (latent_prep), products with one small matrix per
// head (headwise_gemm: qa, and the value up-projection with the output gate in its epilogue),
// and the attention itself.  Norms, angles, scores, the softmax and its sums are 32-bit.
#include "common.cuh"

// ---------------------------------------------------------------------------
// Per token, from the 32-bit down-projections:
//   cq[t, :]  = dq[t, :] / rms * wq                          (query latent, activation type)
//   page row  = [ dkv[t, :rank] / rms * wc | rotate(dkv[t, rank:rank+rot]) ]   at the token's place
// Rotation: entry i of the rot part pairs with entry i + dims/2 (i < dims/2), angle =
// position * inv_freq[i]; entries from `dims` on pass unchanged.
// ---------------------------------------------------------------------------
__global__ void latent_prep_kernel(const float* __restrict__ dq, int ld_dq, const float* __restrict__ dkv,
                                   int ld_dkv, const float* __restrict__ wq, const float* __restrict__ wc,
                                   float eps, act_t* __restrict__ cq, act_t* __restrict__ pages,
                                   const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                                   const int* __restrict__ seq_slot, const int* __restrict__ page_table,
                                   int table_stride, const float* __restrict__ inv_freq, int q_rank, int rank,
                                   int rot, int dims) {
  __shared__ float scratch[33];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const float* a = dq + (size_t)t * ld_dq;
  const float* b = dkv + (size_t)t * ld_dkv;
  float sq = 0.0f, sc = 0.0f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) sq = fmaf(a[i], a[i], sq);
  for (int i = threadIdx.x; i < rank; i += blockDim.x) sc = fmaf(b[i], b[i], sc);
  sq = block_sum(sq, scratch);
  sc = block_sum(sc, scratch);
  const float rq = sqrtf(sq / (float)q_rank + eps), rc = sqrtf(sc / (float)rank + eps);
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
    cq[(size_t)t * q_rank + i] = from_f32<act_t>((a[i] / rq) * wq[i]);
  const int pos = token_pos[t];
  const int page = page_table[(size_t)seq_slot[token_seq[t]] * table_stride + pos / TL_PAGE];
  const int width = rank + rot;
  act_t* row = pages + ((size_t)page * TL_PAGE + (pos % TL_PAGE)) * width;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) row[i] = from_f32<act_t>((b[i] / rc) * wc[i]);
  const int half = dims >> 1;
  const float* r = b + rank;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, cs;
    sincosf((float)pos * inv_freq[i], &sn, &cs);
    const float u = r[i], v = r[i + half];
    row[rank + i] = from_f32<act_t>(u * cs - v * sn);
    row[rank + i + half] = from_f32<act_t>(v * cs + u * sn);
  }
  for (int i = dims + threadIdx.x; i < rot; i += blockDim.x) row[rank + i] = from_f32<act_t>(r[i]);
}

extern "C" int TL_NAME(tl_latent_prep)(const float* dq, int ld_dq, const float* dkv, int ld_dkv, const float* wq,
                                       const float* wc, float eps, void* cq, void* pages, const int* token_pos,
                                       const int* token_seq, const int* seq_slot, const int* page_table,
                                       int table_stride, const float* inv_freq, int T, int q_rank, int rank,
                                       int rot, int dims, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (q_rank <= 0 || rank <= 0 || rot < 0 || dims < 0 || dims > rot || (dims & 1)) return TL_ERR_BAD_ARG;
  return tl_launch(latent_prep_kernel, dim3(T), dim3(128), 0, stream, dq, ld_dq, dkv, ld_dkv, wq, wc, eps,
                   (act_t*)cq, (act_t*)pages, token_pos, token_seq, seq_slot, page_table, table_stride, inv_freq,
                   q_rank, rank, rot, dims);
}

// ---------------------------------------------------------------------------
// One small product per head:  C[t, h, n] = sum_k A[t, h, k] * W[h, n, k]
//   A 32-bit, row stride lda, head h at column h * a_head;  W [heads, N, K] in the activation type;
//   C row stride ldc, head h at column h * c_head.
// epilogue 0: C 32-bit = product;  1: C (activation type) = product * sigmoid(G[t, h * N + n]),
// G 32-bit with row stride ldg (an output gate), or the product alone where G is null.
// 64 x 64 tiles, 16 K-elements a step, 256 threads with 4 x 4 outputs each; 32-bit FFMA.
// ---------------------------------------------------------------------------
#define HW_BM 64
#define HW_BN 64
#define HW_BK 16

template <int EPI>
__global__ void __launch_bounds__(256)
headwise_gemm_kernel(const float* __restrict__ A, int lda, int a_head, const act_t* __restrict__ W,
                     void* __restrict__ C, int ldc, int c_head, const float* __restrict__ G, int ldg, int M,
                     int N, int K) {
  __shared__ float As[HW_BK][HW_BM + 4];
  __shared__ float Ws[HW_BK][HW_BN + 4];
  pdl_wait();
  pdl_launch_dependents();
  const int h = blockIdx.z;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * HW_BM, n0 = blockIdx.x * HW_BN;
  const float* Ah = A + (size_t)h * a_head;
  const act_t* Wh = W + (size_t)h * N * K;
  float acc[4][4] = {};
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  for (int k0 = 0; k0 < K; k0 += HW_BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lk + j;
      const int am = m0 + lrow, wn = n0 + lrow;
      As[lk + j][lrow] = (am < M && k < K) ? Ah[(size_t)am * lda + k] : 0.0f;
      Ws[lk + j][lrow] = (wn < N && k < K) ? to_f32(Wh[(size_t)wn * K + k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < HW_BK; ++k) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      const size_t at = (size_t)m * ldc + (size_t)h * c_head + n;
      if (EPI == 0) {
        ((float*)C)[at] = acc[i][j];
      } else {
        const float g = G != nullptr ? 1.0f / (1.0f + expf(-G[(size_t)m * ldg + (size_t)h * N + n])) : 1.0f;
        ((act_t*)C)[at] = from_f32<act_t>(acc[i][j] * g);
      }
    }
  }
}

// Few rows (decode): a warp per (row, head, output) streams one row of W.
template <int EPI>
__global__ void __launch_bounds__(256)
headwise_gemv_kernel(const float* __restrict__ A, int lda, int a_head, const act_t* __restrict__ W,
                     void* __restrict__ C, int ldc, int c_head, const float* __restrict__ G, int ldg, int M,
                     int N, int K) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int h = blockIdx.z, m = blockIdx.y;
  if (n >= N) return;
  const float* a = A + (size_t)m * lda + (size_t)h * a_head;
  const act_t* w = W + ((size_t)h * N + n) * K;
  float acc = 0.0f;
  for (int k = lane; k < K; k += 32) acc = fmaf(a[k], to_f32(w[k]), acc);
  acc = warp_sum(acc);
  if (lane == 0) {
    const size_t at = (size_t)m * ldc + (size_t)h * c_head + n;
    if (EPI == 0) {
      ((float*)C)[at] = acc;
    } else {
      const float g = G != nullptr ? 1.0f / (1.0f + expf(-G[(size_t)m * ldg + (size_t)h * N + n])) : 1.0f;
      ((act_t*)C)[at] = from_f32<act_t>(acc * g);
    }
  }
}

extern "C" int TL_NAME(tl_headwise_gemm)(const float* A, int lda, int a_head, const void* W, void* C, int ldc,
                                         int c_head, const float* G, int ldg, int M, int N, int K, int heads,
                                         int epilogue, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || heads <= 0) return 0;
  if (K <= 0 || epilogue < 0 || epilogue > 1) return TL_ERR_BAD_ARG;
  if (heads > 65535) return TL_ERR_UNSUPPORTED;
  if (M <= 16) {
    dim3 grid((N + 7) / 8, M, heads);
    if (epilogue == 0)
      return tl_launch(headwise_gemv_kernel<0>, grid, dim3(256), 0, stream, A, lda, a_head, (const act_t*)W, C,
                       ldc, c_head, G, ldg, M, N, K);
    return tl_launch(headwise_gemv_kernel<1>, grid, dim3(256), 0, stream, A, lda, a_head, (const act_t*)W, C, ldc,
                     c_head, G, ldg, M, N, K);
  }
  dim3 grid((N + HW_BN - 1) / HW_BN, (M + HW_BM - 1) / HW_BM, heads);
  if (grid.y > 65535) return TL_ERR_UNSUPPORTED;
  if (epilogue == 0)
    return tl_launch(headwise_gemm_kernel<0>, grid, dim3(256), 0, stream, A, lda, a_head, (const act_t*)W, C, ldc,
                     c_head, G, ldg, M, N, K);
  return tl_launch(headwise_gemm_kernel<1>, grid, dim3(256), 0, stream, A, lda, a_head, (const act_t*)W, C, ldc,
                   c_head, G, ldg, M, N, K);
}

// ---------------------------------------------------------------------------
// The attention.  One block per (token, head): the query [qa (rank) | rotate(q_rot) (rot)] times
// `scale` lies in shared memory; keys are the page rows of positions max(0, p - W + 1) .. p (W = 0:
// from 0), taken 128 at a time from the first visible one with a running maximum and sum, so a
// position's result is the same in whatever step or batch it is computed.  The weighted sum of
// the rows' first `rank` numbers goes to o[t, h, :] (32-bit).
//   qa [T, ld_qa] 32-bit, head h's latent-space query at h * qa_head;  q [T, ldq] 32-bit, head h's
//   part to rotate at h * q_head + q_off (both may lie in one buffer)
// ---------------------------------------------------------------------------
#define LAT_THREADS 128
#define LAT_MAX_PER_THREAD 8   // rank <= 1024

#if TL_DTYPE == 0
#define LVEC 4
__device__ __forceinline__ void load_row_vec(const act_t* p, float* out) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
#else
#define LVEC 8
__device__ __forceinline__ void load_row_vec(const act_t* p, float* out) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}
#endif

__global__ void __launch_bounds__(LAT_THREADS)
latent_attn_kernel(const float* __restrict__ qa, int ld_qa, int qa_head, const float* __restrict__ q, int ldq,
                   int q_head, int q_off,
                   const act_t* __restrict__ pages, float* __restrict__ o, const int* __restrict__ token_pos,
                   const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
                   const int* __restrict__ page_table, int table_stride, const float* __restrict__ inv_freq,
                   const float* __restrict__ sink, int heads, int rank, int rot, int dims, int window, float scale) {
  extern __shared__ float qs[];          // [rank + rot]
  __shared__ float ps[LAT_THREADS];
  __shared__ int pg[LAT_THREADS];
  __shared__ float scratch[33];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int width = rank + rot;
  const int pos = token_pos[t];
  const int* table = page_table + (size_t)seq_slot[token_seq[t]] * table_stride;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const bool vec = width % LVEC == 0;     // rows then start on 16-byte boundaries
  for (int i = tid; i < rank; i += LAT_THREADS) qs[i] = qa[(size_t)t * ld_qa + (size_t)h * qa_head + i] * scale;
  {
    const float* r = q + (size_t)t * ldq + (size_t)h * q_head + q_off;
    const int half = dims >> 1;
    for (int i = tid; i < half; i += LAT_THREADS) {
      float sn, cs;
      sincosf((float)pos * inv_freq[i], &sn, &cs);
      const float u = r[i], v = r[i + half];
      qs[rank + i] = (u * cs - v * sn) * scale;
      qs[rank + i + half] = (v * cs + u * sn) * scale;
    }
    for (int i = dims + tid; i < rot; i += LAT_THREADS) qs[rank + i] = r[i] * scale;
  }
  __syncthreads();
  float m_run = -INFINITY, l_run = 0.0f;
  float acc[LAT_MAX_PER_THREAD];
#pragma unroll
  for (int j = 0; j < LAT_MAX_PER_THREAD; ++j) acc[j] = 0.0f;
  for (int base = lo; base <= pos; base += LAT_THREADS) {
    const int i = base + tid;
    const bool valid = i <= pos;
    float s = -INFINITY;
    int page = -1;
    if (valid) {
      page = table[i / TL_PAGE];
      const act_t* krow = pages + ((size_t)page * TL_PAGE + (i % TL_PAGE)) * width;
      float dot = 0.0f;
      if (vec) {
        for (int d = 0; d < width; d += LVEC) {
          float kv[LVEC];
          load_row_vec(krow + d, kv);
#pragma unroll
          for (int e = 0; e < LVEC; ++e) dot = fmaf(qs[d + e], kv[e], dot);
        }
      } else {
        for (int d = 0; d < width; ++d) dot = fmaf(qs[d], to_f32(krow[d]), dot);
      }
      s = dot;
    }
    const float cmax = block_max(s, scratch);
    const float m_new = fmaxf(m_run, cmax);
    const float p = valid ? expf(s - m_new) : 0.0f;
    ps[tid] = p;
    pg[tid] = page;
    const float csum = block_sum(p, scratch);   // its barriers publish ps and pg
    const float alpha = expf(m_run - m_new);    // 0 at the first chunk
    l_run = l_run * alpha + csum;
    m_run = m_new;
    const int cnt = (pos - base + 1 < LAT_THREADS) ? pos - base + 1 : LAT_THREADS;
#pragma unroll
    for (int j = 0; j < LAT_MAX_PER_THREAD; ++j) {
      const int d = tid + j * LAT_THREADS;
      if (d < rank) {
        float a = acc[j] * alpha;
        for (int k = 0; k < cnt; ++k) {
          const act_t* vrow = pages + ((size_t)pg[k] * TL_PAGE + ((base + k) % TL_PAGE)) * width;
          a = fmaf(ps[k], to_f32(vrow[d]), a);
        }
        acc[j] = a;
      }
    }
    __syncthreads();   // ps and pg are rewritten by the next chunk
  }
  // a sink is a key with the score sink[h] (not scaled) and no value: it only enters the denominator
  const float denom = sink != nullptr ? l_run + expf(sink[h] - m_run) : l_run;
  float* orow = o + ((size_t)t * heads + h) * rank;
#pragma unroll
  for (int j = 0; j < LAT_MAX_PER_THREAD; ++j) {
    const int d = tid + j * LAT_THREADS;
    if (d < rank) orow[d] = acc[j] / denom;
  }
}

extern "C" int TL_NAME(tl_latent_attn)(const float* qa, int ld_qa, int qa_head, const float* q, int ldq,
                                       int q_head, int q_off,
                                       const void* pages, float* o, const int* token_pos, const int* token_seq,
                                       const int* seq_slot, const int* page_table, int table_stride,
                                       const float* inv_freq, const float* sink, int T, int heads, int rank,
                                       int rot, int dims, int window, float scale, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (heads <= 0 || rank <= 0 || rot < 0 || dims > rot || (dims & 1)) return TL_ERR_BAD_ARG;
  if (rank > LAT_THREADS * LAT_MAX_PER_THREAD || heads > 65535 || (rank + rot) * sizeof(float) > 40 * 1024)
    return TL_ERR_UNSUPPORTED;
  return tl_launch(latent_attn_kernel, dim3(T, heads), dim3(LAT_THREADS), (size_t)(rank + rot) * sizeof(float),
                   stream, qa, ld_qa, qa_head, q, ldq, q_head, q_off, (const act_t*)pages, o, token_pos, token_seq, seq_slot,
                   page_table, table_stride, inv_freq, sink, heads, rank, rot, dims, window, scale);
}

#if TL_DTYPE == 1
// ---------------------------------------------------------------------------
// The same attention on tensor cores (bfloat16 build).  All heads of a token share the keys, so
// the heads are the rows of the tiles: a block takes one token and up to 16 heads, and a part of
// the token's visible keys (`splits` parts; more than one for decode steps, whose few tokens
// would leave most of the GPU idle; a second kernel merges the parts).
//
// Per chunk of 64 keys: the chunk's page rows are copied to shared memory once (cp.async) and
// serve both products.  Scores: each of the 4 warps takes 16 keys, S[16 heads x 16 keys] =
// Q K^T by mma.sync m16n8k16 (Q, rotated and scaled, lies in shared memory as bfloat16), and
// writes them in 32-bit to shared memory.  Softmax: every warp reads all 64 scores of its rows
// in the layout of an A operand, keeps the running maximum and sum in 32-bit (the same numbers in
// every warp), and rounds the weights to bfloat16.  Weighted sum: the warps share the columns of c
// in groups of 16; B operands are read from the same rows with ldmatrix.trans; the sums stay in
// registers (32-bit) over all chunks.
// Needs rank and rot to be multiples of 16 and rank <= 512; other sizes take the kernel above.
// ---------------------------------------------------------------------------
#define LM_KC 64
#define LM_THREADS 128
#define LM_SPITCH (LM_KC + 4)

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
               "{%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x by the hardware's approximation (relative error about 2^-22; 0 for x = -inf), as the other
// tensor-core attention kernels of this package take their exponentials.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// NTP: pairs of 8-column tiles of c per warp (rank <= 64 * NTP).  TB: tokens per block, each with four
// warps of its own; the tokens of a block that belong to one sequence share the key chunks in shared
// memory (neighbouring positions see nearly the same keys), which divides what the block fetches
// from the L2 cache by TB.  Keys are cut into parts (`splits` > 1) only with TB = 1.
template <int NTP, int TB>
__global__ void __launch_bounds__(LM_THREADS * TB)
latent_attn_mma_kernel(const float* __restrict__ qa, int ld_qa, int qa_head, const float* __restrict__ q, int ldq,
                       int q_head, int q_off, const __nv_bfloat16* __restrict__ pages, float* __restrict__ o,
                       float* __restrict__ part, const int* __restrict__ token_pos,
                       const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
                       const int* __restrict__ page_table, int table_stride, const float* __restrict__ inv_freq,
                       const float* __restrict__ sink, int T, int heads, int rank, int rot, int dims, int window,
                       float scale, int splits) {
  extern __shared__ __align__(16) unsigned char lm_smem[];
  const int width = rank + rot, pitch = width + 8;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(lm_smem);          // [TB][16][pitch]
  __nv_bfloat16* Ks = Qs + TB * 16 * pitch;                                // [LM_KC][pitch]
  float* Ss_all = reinterpret_cast<float*>(Ks + LM_KC * pitch);            // [TB][16][LM_SPITCH]
  const __nv_bfloat16** rowp = reinterpret_cast<const __nv_bfloat16**>(Ss_all + TB * 16 * LM_SPITCH);   // [LM_KC]
  __shared__ int s_pos[TB], s_seq[TB];
  pdl_wait();
  pdl_launch_dependents();
  const int t0 = blockIdx.x * TB, split = blockIdx.y, hg = blockIdx.z;
  const int nb = min(TB, T - t0);                  // tokens of this block
  const int tid = threadIdx.x, lane = tid & 31;
  const int wg = tid >> 7, warp = (tid >> 5) & 3;  // the token's place in the block; the warp's among the token's four
  const int g = lane >> 2, qd = lane & 3;
  if (tid < nb) { s_pos[tid] = token_pos[t0 + tid]; s_seq[tid] = token_seq[t0 + tid]; }
  __syncthreads();
  const int my = wg < nb ? wg : nb - 1;            // a group without a token mirrors the last one and writes nothing
  const int pos = s_pos[my];
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  __nv_bfloat16* Qt = Qs + wg * 16 * pitch;
  float* Ss = Ss_all + wg * 16 * LM_SPITCH;
  // the queries of this token's heads: [latent-space part | rotated part], times scale; cosines and sines
  // of the token's angles once per token (they wait in the token's score buffer, which is free until the
  // first chunk)
  {
    const int half = dims >> 1;
    const int t = t0 + my;
    const int tl = tid & (LM_THREADS - 1);
    float2* cs_s = reinterpret_cast<float2*>(Ss);            // [half] <= 16 * LM_SPITCH / 2 (the launcher checks)
    for (int i = tl; i < half; i += LM_THREADS) {
      float sn, cs;
      sincosf((float)pos * inv_freq[i], &sn, &cs);
      cs_s[i] = make_float2(cs, sn);
    }
    __syncthreads();
    const float qscale = scale * 1.4426950408889634f;      // log2(e): the softmax below works in base 2
    // the latent-space parts of four heads at a time: their loads are all issued before the first is used
    // (one after the other they cost a block of one chunk some twenty microseconds)
    for (int r0 = 0; r0 < 16; r0 += 4) {
      float v[4][4];                                   // rank <= 512: at most 4 values a thread and head
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int h = hg * 16 + r0 + j;
        const float* qsrc = qa + (size_t)t * ld_qa + (size_t)(h < heads ? h : 0) * qa_head;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int d = tl + k * LM_THREADS;
          v[j][k] = (h < heads && d < rank) ? qsrc[d] : 0.0f;
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int d = tl + k * LM_THREADS;
          if (d < rank) Qt[(r0 + j) * pitch + d] = __float2bfloat16_rn(v[j][k] * qscale);
        }
    }
    // the parts to rotate: a thread takes one pair of entries of all 16 heads, loads first
    for (int i = tl; i < half; i += LM_THREADS) {
      float u[16], w[16];
#pragma unroll
      for (int r = 0; r < 16; ++r) {
        const int h = hg * 16 + r;
        const float* src = q + (size_t)t * ldq + (size_t)(h < heads ? h : 0) * q_head + q_off;
        u[r] = h < heads ? src[i] : 0.0f;
        w[r] = h < heads ? src[i + half] : 0.0f;
      }
      const float2 c = cs_s[i];
#pragma unroll
      for (int r = 0; r < 16; ++r) {
        Qt[r * pitch + rank + i] = __float2bfloat16_rn((u[r] * c.x - w[r] * c.y) * qscale);
        Qt[r * pitch + rank + half + i] = __float2bfloat16_rn((w[r] * c.x + u[r] * c.y) * qscale);
      }
    }
    for (int j = dims + tl; j < rot; j += LM_THREADS) {      // entries that pass unrotated
#pragma unroll
      for (int r = 0; r < 16; ++r) {
        const int h = hg * 16 + r;
        const float x = h < heads ? q[(size_t)t * ldq + (size_t)h * q_head + q_off + j] : 0.0f;
        Qt[r * pitch + rank + j] = __float2bfloat16_rn(x * qscale);
      }
    }
  }
  float acc[2 * NTP][4];
#pragma unroll
  for (int i = 0; i < 2 * NTP; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};   // rows g and g + 8
  const int n_pairs = rank >> 4;        // groups of 16 columns of c
  const int vecs = width >> 3;          // 16-byte pieces per row
  // runs of tokens of one sequence (a block may straddle the end of a sequence of the packed batch)
  for (int r_begin = 0; r_begin < nb;) {
    int r_end = r_begin + 1;
    while (r_end < nb && s_seq[r_end] == s_seq[r_begin]) ++r_end;
    const bool active = wg >= r_begin && wg < r_end;
    const int* table = page_table + (size_t)seq_slot[s_seq[r_begin]] * table_stride;
    const int p_first = s_pos[r_begin], p_last = s_pos[r_end - 1];
    const int lo_min = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
    const int n_chunks = (p_last - lo_min + LM_KC) / LM_KC;
    const int per_split = (n_chunks + splits - 1) / splits;
    const int c_begin = split * per_split;
    const int c_end = min(n_chunks, c_begin + per_split);
    for (int c = c_begin; c < c_end; ++c) {
      const int base = lo_min + c * LM_KC;
      __syncthreads();     // the chunk before is done with Ks, Ss and rowp (and Qs is written)
      if (tid < LM_KC) {
        const int i = base + tid;
        rowp[tid] = i <= p_last ? pages + ((size_t)table[i / TL_PAGE] * TL_PAGE + (i % TL_PAGE)) * width : nullptr;
      }
      __syncthreads();
      if (TB == 1) {
        // a warp copies whole rows, 512 bytes an instruction (no index is divided: with one warp per
        // scheduler every instruction counts)
        for (int r = tid >> 5; r < LM_KC; r += LM_THREADS / 32) {
          const __nv_bfloat16* src = rowp[r];
          __nv_bfloat16* dst = Ks + r * pitch;
          if (src != nullptr) {
            for (int v = lane; v < vecs; v += 32) {
              const uint32_t d32 = (uint32_t)__cvta_generic_to_shared(dst + v * 8);
              asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d32), "l"(src + v * 8) : "memory");
            }
          } else {
            for (int v = lane; v < vecs; v += 32) *reinterpret_cast<uint4*>(dst + v * 8) = make_uint4(0u, 0u, 0u, 0u);
          }
        }
      } else {
        // a fixed row per thread (2 TB threads share a row, 32 TB bytes in a run), so that no index is
        // divided (measured at four tokens a block: 747 us against 838 us with the loop above and 823 us
        // with a warp per row)
        constexpr int PER_ROW = LM_THREADS * TB / LM_KC;
        const int r = tid / PER_ROW;
        const __nv_bfloat16* src = rowp[r];
        __nv_bfloat16* dst = Ks + r * pitch;
        if (src != nullptr) {
          for (int v = tid % PER_ROW; v < vecs; v += PER_ROW) {
            const uint32_t d32 = (uint32_t)__cvta_generic_to_shared(dst + v * 8);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d32), "l"(src + v * 8) : "memory");
          }
        } else {
          for (int v = tid % PER_ROW; v < vecs; v += PER_ROW)
            *reinterpret_cast<uint4*>(dst + v * 8) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      asm volatile("cp.async.commit_group;\n cp.async.wait_group 0;" ::: "memory");
      __syncthreads();
      // scores of this warp's 16 keys
      if (active) {
        float sc[2][4] = {};
        const __nv_bfloat16* qrow = Qt + ((lane & 7) + ((lane >> 3) & 1) * 8) * pitch + (lane >> 4) * 8;
        const __nv_bfloat16* krow = Ks + (warp * 16 + (lane >> 4) * 8 + (lane & 7)) * pitch + ((lane >> 3) & 1) * 8;
        // (unrolled so that the loads of the next steps are issued before this step's products wait for theirs)
#pragma unroll 4
        for (int ks = 0; ks < width; ks += 16) {
          uint32_t a[4], b[4];
          ldsm_x4(a, qrow + ks);
          ldsm_x4(b, krow + ks);
          mma_bf16(sc[0], a, b[0], b[1]);
          mma_bf16(sc[1], a, b[2], b[3]);
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const int col = warp * 16 + nt * 8 + qd * 2;
          const int k0 = base + col;
          const bool v0 = k0 >= lo && k0 <= pos, v1 = k0 + 1 >= lo && k0 + 1 <= pos;
          Ss[g * LM_SPITCH + col] = v0 ? sc[nt][0] : -INFINITY;
          Ss[g * LM_SPITCH + col + 1] = v1 ? sc[nt][1] : -INFINITY;
          Ss[(g + 8) * LM_SPITCH + col] = v0 ? sc[nt][2] : -INFINITY;
          Ss[(g + 8) * LM_SPITCH + col + 1] = v1 ? sc[nt][3] : -INFINITY;
        }
      }
      __syncthreads();
      if (!active) continue;
      // softmax over the chunk, per row; the weights as A operands of the second product
      float s[2][LM_KC / 16][4];
      float cmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int kk = 0; kk < LM_KC / 16; ++kk) {
          const float2 x = *reinterpret_cast<const float2*>(Ss + (g + 8 * r) * LM_SPITCH + kk * 16 + qd * 2);
          const float2 y = *reinterpret_cast<const float2*>(Ss + (g + 8 * r) * LM_SPITCH + kk * 16 + 8 + qd * 2);
          s[r][kk][0] = x.x; s[r][kk][1] = x.y; s[r][kk][2] = y.x; s[r][kk][3] = y.y;
          cmax[r] = fmaxf(cmax[r], fmaxf(fmaxf(x.x, x.y), fmaxf(y.x, y.y)));
        }
      float alpha[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        cmax[r] = fmaxf(cmax[r], __shfl_xor_sync(0xffffffffu, cmax[r], 1));
        cmax[r] = fmaxf(cmax[r], __shfl_xor_sync(0xffffffffu, cmax[r], 2));
        // The first chunk of a token's range holds a key it sees, so the maximum is finite from then on; a
        // later chunk in which this token sees no key (only a neighbour does) leaves everything as it is.
        const float m_new = fmaxf(m_run[r], cmax[r]);
        alpha[r] = m_new == -INFINITY ? 1.0f : fast_exp2(m_run[r] - m_new);      // 0 at the first chunk
        float sum = 0.0f;
#pragma unroll
        for (int kk = 0; kk < LM_KC / 16; ++kk)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            s[r][kk][e] = m_new == -INFINITY ? 0.0f : fast_exp2(s[r][kk][e] - m_new);   // 0 for keys not seen
            sum += s[r][kk][e];
          }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        l_run[r] = l_run[r] * alpha[r] + sum;
        m_run[r] = m_new;
      }
#pragma unroll
      for (int i = 0; i < 2 * NTP; ++i) {
        acc[i][0] *= alpha[0]; acc[i][1] *= alpha[0];
        acc[i][2] *= alpha[1]; acc[i][3] *= alpha[1];
      }
#pragma unroll
      for (int kk = 0; kk < LM_KC / 16; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[0][kk][0], s[0][kk][1]);
        a[1] = pack_bf16(s[1][kk][0], s[1][kk][1]);
        a[2] = pack_bf16(s[0][kk][2], s[0][kk][3]);
        a[3] = pack_bf16(s[1][kk][2], s[1][kk][3]);
        const __nv_bfloat16* vrow = Ks + (kk * 16 + (lane & 15)) * pitch + (lane >> 4) * 8;
#pragma unroll
        for (int i = 0; i < NTP; ++i) {
          const int pair = warp + 4 * i;
          if (pair < n_pairs) {
            uint32_t b[4];
            ldsm_x4_trans(b, vrow + pair * 16);
            mma_bf16(acc[2 * i], a, b[0], b[1]);
            mma_bf16(acc[2 * i + 1], a, b[2], b[3]);
          }
        }
      }
    }
    r_begin = r_end;
  }
  if (wg >= nb) return;
  // out: normalised if this block saw all the keys, else this part's sums with its maximum and sum
  const int t = t0 + wg;
  const int hpad = gridDim.z * 16;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = hg * 16 + g + 8 * r;
    if (splits == 1) {
      if (row >= heads) continue;
      // a sink only enters the denominator (the running maximum is that of the scores times log2(e))
      const float inv = 1.0f / (sink != nullptr ? l_run[r] + exp2f(sink[row] * 1.4426950408889634f - m_run[r])
                                                : l_run[r]);
      float* dst = o + ((size_t)t * heads + row) * rank;
#pragma unroll
      for (int i = 0; i < NTP; ++i) {
        const int pair = warp + 4 * i;
        if (pair < n_pairs) {
#pragma unroll
          for (int j = 0; j < 2; ++j)
            *reinterpret_cast<float2*>(dst + pair * 16 + j * 8 + qd * 2) =
                make_float2(acc[2 * i + j][2 * r] * inv, acc[2 * i + j][2 * r + 1] * inv);
        }
      }
    } else {
      float* dst = part + (((size_t)t * hpad + row) * splits + split) * (size_t)(rank + 2);
#pragma unroll
      for (int i = 0; i < NTP; ++i) {
        const int pair = warp + 4 * i;
        if (pair < n_pairs) {
#pragma unroll
          for (int j = 0; j < 2; ++j)
            *reinterpret_cast<float2*>(dst + pair * 16 + j * 8 + qd * 2) =
                make_float2(acc[2 * i + j][2 * r], acc[2 * i + j][2 * r + 1]);
        }
      }
      if (warp == 0 && qd == 0) { dst[rank] = m_run[r]; dst[rank + 1] = l_run[r]; }
    }
  }
}

// Merges the parts of a token's keys: out = sum_s w_s O_s / sum_s w_s l_s with w_s = 2^(m_s - max m)
// (the maxima are those of the scores times log2(e)).
__global__ void __launch_bounds__(128)
latent_attn_merge_kernel(const float* __restrict__ part, float* __restrict__ o, const float* __restrict__ sink,
                         int heads, int hpad, int rank, int splits) {
  __shared__ float w_s[64];      // the parts' weights (at most 64 parts), then divided by their sum
  __shared__ float scratch[33];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, h = blockIdx.y;
  const size_t stride = (size_t)(rank + 2);
  const float* src = part + ((size_t)t * hpad + h) * splits * stride;
  const float ms = (int)threadIdx.x < splits ? src[threadIdx.x * stride + rank] : -INFINITY;
  const float sink2 = sink != nullptr ? sink[h] * 1.4426950408889634f : -INFINITY;
  const float m = fmaxf(block_max(ms, scratch), sink2);
  const float w = ms != -INFINITY ? exp2f(ms - m) : 0.0f;
  float l = block_sum((int)threadIdx.x < splits ? w * src[threadIdx.x * stride + rank + 1] : 0.0f, scratch);
  if (sink != nullptr) l += exp2f(sink2 - m);        // the sink is counted once, whatever the parts
  if ((int)threadIdx.x < splits) w_s[threadIdx.x] = w / l;
  __syncthreads();
  for (int d = threadIdx.x; d < rank; d += blockDim.x) {
    float a = 0.0f;
#pragma unroll 8
    for (int s = 0; s < splits; ++s) a = fmaf(w_s[s], src[(size_t)s * stride + d], a);
    o[((size_t)t * heads + h) * rank + d] = a;
  }
}

// How many parts the keys of a step's tokens are cut into, and how many floats the parts need.
// `max_keys`: an upper bound of the keys any token of the step sees.
extern "C" int tl_latent_attn_plan(int T, int heads, int rank, int rot, int max_keys, int num_sms,
                                   long long* part_floats) {
  *part_floats = 0;
  if (rank % 16 || rot % 16 || rank > 512 || rank <= 0 || rot > 1024) return 0;     // the CUDA-core kernel
  const size_t smem = (size_t)(16 + LM_KC) * (rank + rot + 8) * 2 + 16 * LM_SPITCH * 4 + LM_KC * 8;
  if (smem > 200 * 1024) return 0;      // (one token a block; lm_smem_bytes(1, ...) below)
  const int groups = (heads + 15) / 16;
  const long long blocks = (long long)T * groups;
  int splits = 1;
  const int chunks = (max_keys + LM_KC - 1) / LM_KC;
  if (blocks < 1LL * num_sms) {
    splits = (int)((1LL * num_sms + blocks - 1) / blocks);
    if (splits > chunks) splits = chunks;
    if (splits > 64) splits = 64;
    if (splits < 1) splits = 1;
  }
  if (splits > 1) *part_floats = (long long)T * groups * 16 * splits * (rank + 2);
  return splits;
}

static size_t lm_smem_bytes(int tb, int rank, int rot) {
  return (size_t)(16 * tb + LM_KC) * (rank + rot + 8) * 2 + (size_t)tb * 16 * LM_SPITCH * 4 + LM_KC * 8;
}

extern "C" int tl_latent_attn_mma(const float* qa, int ld_qa, int qa_head, const float* q, int ldq, int q_head,
                                  int q_off, const void* pages, float* o, float* part, const int* token_pos,
                                  const int* token_seq, const int* seq_slot, const int* page_table,
                                  int table_stride, const float* inv_freq, const float* sink, int T, int heads,
                                  int rank, int rot, int dims, int window, float scale, int splits,
                                  cudaStream_t stream) {
  if (T <= 0) return 0;
  if (rank % 16 || rot % 16 || rank > 512 || rank <= 0 || dims > rot || (dims & 1) || rot > 1024 || splits < 1 ||
      (splits > 1 && part == nullptr))
    return TL_ERR_UNSUPPORTED;
  const int groups = (heads + 15) / 16;
  if (splits > 65535 || groups > 65535) return TL_ERR_UNSUPPORTED;
  // four tokens a block where there are tokens enough to fill the GPU that way and the block fits
  const bool many = splits == 1 && (long long)T * groups >= 8LL * 148 && lm_smem_bytes(4, rank, rot) <= 200 * 1024;
  const int tb = many ? 4 : 1;
  const size_t smem = lm_smem_bytes(tb, rank, rot);
  dim3 grid((T + tb - 1) / tb, splits, groups);
  int rc;
#define LM_LAUNCH_TB(NTP, TBV)                                                                               \
  {                                                                                                          \
    static bool set = false;                                                                                 \
    if (!set) {                                                                                              \
      if (cudaFuncSetAttribute(latent_attn_mma_kernel<NTP, TBV>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                               200 * 1024) != cudaSuccess)                                                   \
        return TL_ERR_UNSUPPORTED;                                                                           \
      set = true;                                                                                            \
    }                                                                                                        \
    rc = tl_launch(latent_attn_mma_kernel<NTP, TBV>, grid, dim3(LM_THREADS * TBV), smem, stream, qa, ld_qa,  \
                   qa_head, q, ldq, q_head, q_off, (const __nv_bfloat16*)pages, o, part, token_pos, token_seq, \
                   seq_slot, page_table, table_stride, inv_freq, sink, T, heads, rank, rot, dims, window,    \
                   scale, splits);                                                                                  \
  }
#define LM_LAUNCH(NTP) \
  { if (many) LM_LAUNCH_TB(NTP, 4) else LM_LAUNCH_TB(NTP, 1) }
  if (rank <= 64) LM_LAUNCH(1)
  else if (rank <= 128) LM_LAUNCH(2)
  else if (rank <= 256) LM_LAUNCH(4)
  else LM_LAUNCH(8)
#undef LM_LAUNCH
#undef LM_LAUNCH_TB
  if (rc != 0 || splits == 1) return rc;
  return tl_launch(latent_attn_merge_kernel, dim3(T, heads), dim3(128), 0, stream, (const float*)part, o, sink,
                   heads, groups * 16, rank, splits);
}

// ---------------------------------------------------------------------------
// The per-head value up-projection with the output gate on tensor cores (bfloat16 build), for steps of
// many tokens:  C[t, h, n] = sigmoid(G[t, h N + n]) * sum_k A[t, h, k] W[h, n, k],  A 32-bit (rounded to
// bfloat16 on its way into shared memory), W and C bfloat16.  A block computes 64 rows x 64 outputs of
// one head; each of its four warps 16 rows; K goes in steps of 32 through shared memory.
// ---------------------------------------------------------------------------
#define HM_BM 64
#define HM_BN 64
#define HM_BK 32
#define HM_PITCH (HM_BK + 8)

__global__ void __launch_bounds__(128)
headwise_mma_kernel(const float* __restrict__ A, int lda, int a_head, const __nv_bfloat16* __restrict__ W,
                    __nv_bfloat16* __restrict__ C, int ldc, int c_head, const float* __restrict__ G, int ldg,
                    int M, int N, int K) {
  __shared__ __align__(16) __nv_bfloat16 As[HM_BM * HM_PITCH];
  __shared__ __align__(16) __nv_bfloat16 Ws[HM_BN * HM_PITCH];
  pdl_wait();
  pdl_launch_dependents();
  const int h = blockIdx.z, m0 = blockIdx.y * HM_BM, n0 = blockIdx.x * HM_BN;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, qd = lane & 3;
  const float* Ah = A + (size_t)h * a_head;
  const __nv_bfloat16* Wh = W + (size_t)h * N * K;
  float acc[HM_BN / 8][4];
#pragma unroll
  for (int i = 0; i < HM_BN / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
  for (int k0 = 0; k0 < K; k0 += HM_BK) {
    __syncthreads();     // the step before has read both tiles
#pragma unroll
    for (int i = 0; i < 4; ++i) {                      // A: 64 rows x 8 pieces of four 32-bit numbers
      const int idx = tid + i * 128, r = idx >> 3, c4 = (idx & 7) * 4;
      float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (m0 + r < M && k0 + c4 < K) v = *reinterpret_cast<const float4*>(Ah + (size_t)(m0 + r) * lda + k0 + c4);
      uint2 u;
      u.x = pack_bf16(v.x, v.y);
      u.y = pack_bf16(v.z, v.w);
      *reinterpret_cast<uint2*>(As + r * HM_PITCH + c4) = u;
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {                      // W: 64 rows x 4 pieces of eight bfloat16
      const int idx = tid + i * 128, r = idx >> 2, c8 = (idx & 3) * 8;
      __nv_bfloat16* dst = Ws + r * HM_PITCH + c8;
      if (n0 + r < N && k0 + c8 < K) {
        const uint32_t d32 = (uint32_t)__cvta_generic_to_shared(dst);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d32), "l"(Wh + (size_t)(n0 + r) * K + k0 + c8)
                     : "memory");
      } else {
        *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    asm volatile("cp.async.commit_group;\n cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < HM_BK; ks += 16) {
      uint32_t a[4];
      ldsm_x4(a, As + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * HM_PITCH + ks + (lane >> 4) * 8);
#pragma unroll
      for (int np = 0; np < HM_BN / 16; ++np) {
        uint32_t b[4];
        ldsm_x4(b, Ws + (np * 16 + (lane >> 4) * 8 + (lane & 7)) * HM_PITCH + ks + ((lane >> 3) & 1) * 8);
        mma_bf16(acc[2 * np], a, b[0], b[1]);
        mma_bf16(acc[2 * np + 1], a, b[2], b[3]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int m = m0 + warp * 16 + g + 8 * r;
    if (m >= M) continue;
#pragma unroll
    for (int nt = 0; nt < HM_BN / 8; ++nt) {
      const int n = n0 + nt * 8 + qd * 2;
      if (n >= N) continue;          // N is even (checked by the launcher), so n + 1 < N too
      float v0 = acc[nt][2 * r], v1 = acc[nt][2 * r + 1];
      if (G != nullptr) {
        const float2 gt = *reinterpret_cast<const float2*>(G + (size_t)m * ldg + (size_t)h * N + n);
        v0 *= 1.0f / (1.0f + expf(-gt.x));
        v1 *= 1.0f / (1.0f + expf(-gt.y));
      }
      *reinterpret_cast<uint32_t*>(C + (size_t)m * ldc + (size_t)h * c_head + n) = pack_bf16(v0, v1);
    }
  }
}

// Returns TL_ERR_UNSUPPORTED for sizes or alignments it does not take (the FFMA kernel then runs).
extern "C" int tl_headwise_mma(const float* A, int lda, int a_head, const void* W, void* C, int ldc, int c_head,
                               const float* G, int ldg, int M, int N, int K, int heads, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || heads <= 0) return 0;
  if (K % 8 || N % 2 || lda % 4 || a_head % 4 || ldc % 2 || c_head % 2 || ldg % 2 ||
      ((uintptr_t)A & 15) || ((uintptr_t)W & 15) || ((uintptr_t)C & 3) || ((uintptr_t)G & 7) || heads > 65535 ||
      (M + HM_BM - 1) / HM_BM > 65535)
    return TL_ERR_UNSUPPORTED;
  dim3 grid((N + HM_BN - 1) / HM_BN, (M + HM_BM - 1) / HM_BM, heads);
  return tl_launch(headwise_mma_kernel, grid, dim3(128), 0, stream, A, lda, a_head, (const __nv_bfloat16*)W,
                   (__nv_bfloat16*)C, ldc, c_head, G, ldg, M, N, K);
}
#endif
