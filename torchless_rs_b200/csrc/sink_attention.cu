// Softmax attention with grouped key/value heads whose scores are capped, whose window keeps the
// sequence's first keys, and whose denominator holds a learned "sink" logit per head; queries and
// keys are RMS-normed per head, the key and value sizes may differ, and every head's output is
// multiplied by a sigmoid gate.  CUDA cores; serves the true 32-bit path and every size.
//
//   score(i, j) = cap * tanh((q_i . k_j) * scale / cap)            (cap 0: no cap)
//   j is visible to i  iff  j <= i and (i - j < window or j < keep_first)   (window 0: every j <= i)
//   p(i, j) = exp(score) / (sum over visible j' of exp(score(i, j')) + exp(sink_h))
//   out_i = gate_i * sum_j p(i, j) v_j
//
// Keys and values come from the paged cache only (keys [page][kv head][TL_PAGE][dim], values
// transposed [page][kv head][vdim][TL_PAGE]); the step's own keys are written there first, so a
// position's result does not depend on the step or batch that computes it.
#include "common.cuh"

#define SA_THREADS 128
#define SA_MAX_DIM 512

// The step's projections (32-bit, one row per token: q heads, k heads, v heads side by side) get
// their biases; q and k are divided by their root mean square per head and multiplied by a weight
// vector shared by the heads; q goes to `q_out` (act_t), k and v into the token's place in the pages.
__global__ void __launch_bounds__(256)
qk_norm_cache_write_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ bias,
                           const float* __restrict__ qw, const float* __restrict__ kw, float eps,
                           act_t* __restrict__ q_out, act_t* __restrict__ k_pages, act_t* __restrict__ v_pages,
                           const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                           const int* __restrict__ seq_slot, const int* __restrict__ page_table,
                           int table_stride, int nh, int nkv, int dim, int vdim) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int pos = token_pos[t];
  const int slot = seq_slot[token_seq[t]];
  const int page = page_table[(size_t)slot * table_stride + pos / TL_PAGE];
  const int in_page = pos % TL_PAGE;
  const float* row = z + (size_t)t * ldz;
  const int k_off = nh * dim, v_off = (nh + nkv) * dim;
  // a warp per head; the heads of a token are spread over the blocks of a grid row
  for (int head = blockIdx.y * nwarps + warp; head < nh + 2 * nkv; head += gridDim.y * nwarps) {
    if (head < nh + nkv) {
      const bool is_q = head < nh;
      const int off = head * dim;                      // q heads, then k heads
      const float* w = is_q ? qw : kw;
      float ss = 0.0f;
      for (int d = lane; d < dim; d += 32) {
        const float v = row[off + d] + (bias != nullptr ? bias[off + d] : 0.0f);
        ss = fmaf(v, v, ss);
      }
      ss = warp_sum(ss);
      const float inv = w != nullptr ? 1.0f / sqrtf(ss / (float)dim + eps) : 1.0f;
      act_t* dst = is_q ? q_out + (size_t)t * nh * dim + (size_t)head * dim
                        : k_pages + (((size_t)page * nkv + (head - nh)) * TL_PAGE + in_page) * dim;
      for (int d = lane; d < dim; d += 32) {
        const float v = row[off + d] + (bias != nullptr ? bias[off + d] : 0.0f);
        dst[d] = from_f32<act_t>(w != nullptr ? v * inv * w[d] : v);
      }
    } else {
      const int g = head - nh - nkv;
      const int off = v_off + g * vdim;
      act_t* dst = v_pages + ((size_t)page * nkv + g) * vdim * TL_PAGE + in_page;
      for (int d = lane; d < vdim; d += 32)
        dst[(size_t)d * TL_PAGE] = from_f32<act_t>(row[off + d] + (bias != nullptr ? bias[off + d] : 0.0f));
    }
  }
  (void)k_off;
}

extern "C" int TL_NAME(tl_qk_norm_cache_write)(const float* z, int ldz, const float* bias, const float* qw,
                                               const float* kw, float eps, void* q_out, void* k_pages,
                                               void* v_pages, const int* token_pos, const int* token_seq,
                                               const int* seq_slot, const int* page_table, int table_stride,
                                               int T, int nh, int nkv, int dim, int vdim, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (nh < 1 || nkv < 1 || dim < 1 || vdim < 1) return TL_ERR_BAD_ARG;
  // few tokens: a block of four warps per four heads, so that a token's heads are worked on at once; many
  // tokens: a block per token
  const int heads = nh + 2 * nkv;
  const bool few = T < 512;
  const dim3 grid(T, few ? (heads + 3) / 4 : 1);
  return tl_launch(qk_norm_cache_write_kernel, grid, dim3(few ? 128 : 256), 0, stream, z, ldz, bias, qw, kw, eps,
                   (act_t*)q_out, (act_t*)k_pages, (act_t*)v_pages, token_pos, token_seq, seq_slot, page_table,
                   table_stride, nh, nkv, dim, vdim);
}

// One block per (token, query head).  The visible keys are walked as one run of n1 + n2 places:
// the n1 kept first keys that lie before the window, then the n2 keys of the window; 128 at a
// time with a running maximum and sum in 32-bit.  The sink opens the running maximum and the
// sum (as a key with score `sink` and no value), so it is counted once whatever the chunks.
__global__ void __launch_bounds__(SA_THREADS)
sink_attn_kernel(const act_t* __restrict__ q, const act_t* __restrict__ k_pages, const act_t* __restrict__ v_pages,
                 const float* __restrict__ gate, int ldg, const float* __restrict__ sink,
                 act_t* __restrict__ out, const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                 const int* __restrict__ seq_slot, const int* __restrict__ page_table, int table_stride, int nh,
                 int nkv, int dim, int vdim, int window, int keep_first, float scale, float cap) {
  __shared__ float qs[SA_MAX_DIM];
  __shared__ float ps[SA_THREADS];
  __shared__ int pg[SA_THREADS];   // page of each key of the chunk
  __shared__ int ky[SA_THREADS];   // its place in the page
  __shared__ float scratch[33];
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int kvh = h / (nh / nkv);
  const int pos = token_pos[t];
  const int slot = seq_slot[token_seq[t]];
  const int* table = page_table + (size_t)slot * table_stride;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int n1 = keep_first < lo ? keep_first : lo;
  const int total = n1 + (pos - lo + 1);
  const size_t kpage = (size_t)nkv * TL_PAGE * dim, vpage = (size_t)nkv * TL_PAGE * vdim;
  const size_t khead = (size_t)kvh * TL_PAGE * dim, vhead = (size_t)kvh * TL_PAGE * vdim;
  const float inv_cap = cap > 0.0f ? 1.0f / cap : 0.0f;

  for (int d = tid; d < dim; d += SA_THREADS) qs[d] = to_f32(q[(size_t)t * nh * dim + (size_t)h * dim + d]);
  __syncthreads();

  float m_run = sink != nullptr ? sink[h] : -INFINITY;
  float l_run = sink != nullptr ? 1.0f : 0.0f;
  float acc0 = 0.0f, acc1 = 0.0f;  // value entries tid and tid + 128
  for (int base = 0; base < total; base += SA_THREADS) {
    const int place = base + tid;
    const bool valid = place < total;
    float s = -INFINITY;
    int page = -1, in_page = 0;
    if (valid) {
      const int key = place < n1 ? place : lo + (place - n1);
      page = table[key / TL_PAGE];
      in_page = key % TL_PAGE;
      const act_t* krow = k_pages + (size_t)page * kpage + khead + (size_t)in_page * dim;
      float dot = 0.0f;
      for (int d = 0; d < dim; ++d) dot = fmaf(qs[d], to_f32(krow[d]), dot);
      s = dot * scale;
      if (cap > 0.0f) s = cap * tanhf(s * inv_cap);
    }
    const float cmax = block_max(s, scratch);
    const float m_new = fmaxf(m_run, cmax);
    const float p = valid ? expf(s - m_new) : 0.0f;
    ps[tid] = p;
    pg[tid] = page;
    ky[tid] = in_page;
    const float csum = block_sum(p, scratch);  // has the barriers that publish ps, pg and ky
    const float alpha = expf(m_run - m_new);   // 0 at the first chunk if there is no sink
    l_run = l_run * alpha + csum;
    m_run = m_new;
    const int cnt = total - base < SA_THREADS ? total - base : SA_THREADS;
    if (tid < vdim) {
      acc0 *= alpha;
      acc1 *= alpha;
      const bool two = tid + SA_THREADS < vdim;
      for (int j = 0; j < cnt; ++j) {
        const act_t* vcol = v_pages + (size_t)pg[j] * vpage + vhead + ky[j];
        const float pj = ps[j];
        acc0 = fmaf(pj, to_f32(vcol[(size_t)tid * TL_PAGE]), acc0);
        if (two) acc1 = fmaf(pj, to_f32(vcol[(size_t)(tid + SA_THREADS) * TL_PAGE]), acc1);
      }
    }
    __syncthreads();  // ps, pg and ky are rewritten by the next chunk
  }
  pdl_launch_dependents();   // only now: a grid let go earlier would sit on the SMs and take issue slots
  float gv = 1.0f;
  if (gate != nullptr) gv = 1.0f / (1.0f + expf(-gate[(size_t)t * ldg + h]));
  const float f = gv / l_run;
  act_t* o = out + (size_t)t * nh * vdim + (size_t)h * vdim;
  if (tid < vdim) o[tid] = from_f32<act_t>(acc0 * f);
  if (tid + SA_THREADS < vdim) o[tid + SA_THREADS] = from_f32<act_t>(acc1 * f);
}

extern "C" int TL_NAME(tl_sink_attn)(const void* q, const void* k_pages, const void* v_pages, const float* gate,
                                     int ldg, const float* sink, void* out, const int* token_pos,
                                     const int* token_seq, const int* seq_slot, const int* page_table,
                                     int table_stride, int T, int nh, int nkv, int dim, int vdim, int window,
                                     int keep_first, float scale, float cap, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (dim < 1 || dim > SA_MAX_DIM || vdim < 1 || vdim > 2 * SA_THREADS || nkv <= 0 || nh % nkv != 0 ||
      nh > 65535 || window < 0 || keep_first < 0)
    return TL_ERR_UNSUPPORTED;
  dim3 grid(T, nh);
  return tl_launch(sink_attn_kernel, grid, dim3(SA_THREADS), 0, stream, (const act_t*)q, (const act_t*)k_pages,
                   (const act_t*)v_pages, gate, ldg, sink, (act_t*)out, token_pos, token_seq, seq_slot,
                   page_table, table_stride, nh, nkv, dim, vdim, window, keep_first, scale, cap);
}
