// What stands around the paged attention kernels for mixers whose queries and keys are rotated
// by position: the step's projections on their way into the cache, and two ways of closing a
// head's output (the difference of two attention maps; a gate per output entry).
//
//   rotary_cache_write   z (32-bit rows: query vectors, key vectors, value heads side by side)
//                        -> rotated (and, if asked, unit-normed) q in the activation type, rotated
//                        k and plain v into the token's place in the pages.
//   diff_heads           o = a1 - lambda a2 per head, o / rms(o) * mult.
//   sigmoid_gate         out *= sigmoid(gate), entry by entry.
//
// Rotation: the first `rot` entries of a vector turn in pairs by the angle pos * inv_freq[i],
// pair i being (i, i + rot/2) (style 0) or (2i, 2i + 1) (style 1); the other entries pass.  Angle,
// sine and cosine are 32-bit.
//
// Several maps per head ("slots"): a key/value head's key row in the pages is its `slots` key
// vectors side by side (slots * dim numbers), and query vector j is written as a row of the same
// width that is zero outside slot j % slots.  The dot product of such a query with a key row is
// that of the query with its own map's key, so an attention kernel that knows nothing of maps
// computes every map as a query head of its own over the group's one value head.
#include "common.cuh"

#define RA_MAX_DIM 256
#define RA_WARPS 4

__global__ void __launch_bounds__(RA_WARPS * 32)
rotary_cache_write_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ inv_freq, int rot,
                          int style, int unit_norm, float eps, act_t* __restrict__ q_out,
                          act_t* __restrict__ k_pages, act_t* __restrict__ v_pages,
                          const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                          const int* __restrict__ seq_slot, const int* __restrict__ page_table,
                          int table_stride, int nq, int nk, int nv, int dim, int vdim, int slots) {
  __shared__ float vec[RA_WARPS][RA_MAX_DIM];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pos = token_pos[t];
  const int slot = seq_slot[token_seq[t]];
  const int page = page_table[(size_t)slot * table_stride + pos / TL_PAGE];
  const int in_page = pos % TL_PAGE;
  const float* row = z + (size_t)t * ldz;
  const int half = rot / 2;
  const int width = slots * dim;            // of a query row and of a key row in the pages
  const int nkv = nk / slots;
  const float fpos = (float)pos;
  float* mine = vec[warp];
  // a warp per vector; a token's vectors are spread over the blocks of a grid row
  for (int j = blockIdx.y * RA_WARPS + warp; j < nq + nk + nv; j += gridDim.y * RA_WARPS) {
    if (j < nq + nk) {
      const float* src = row + (size_t)j * dim;
      for (int d = lane; d < dim; d += 32) mine[d] = src[d];
      __syncwarp();
      float ss = 0.0f;
      float keep[RA_MAX_DIM / 32];
#pragma unroll
      for (int r = 0; r < RA_MAX_DIM / 32; ++r) {
        const int d = lane + 32 * r;
        float v = 0.0f;
        if (d < dim) {
          v = mine[d];
          if (d < rot) {
            int i, partner;
            bool first;
            if (style == 0) {
              first = d < half;
              i = first ? d : d - half;
              partner = first ? d + half : d - half;
            } else {
              first = (d & 1) == 0;
              i = d >> 1;
              partner = d ^ 1;
            }
            const float a = fpos * inv_freq[i];
            float sn, cs;
            sincosf(a, &sn, &cs);
            const float o = mine[partner];
            // (u, v) -> (u cos - v sin, v cos + u sin)
            v = first ? v * cs - o * sn : v * cs + o * sn;
          }
        }
        keep[r] = v;
        ss = fmaf(v, v, ss);
      }
      float inv = 1.0f;
      if (unit_norm) {
        ss = warp_sum(ss);
        inv = 1.0f / sqrtf(ss / (float)dim + eps);
      }
      const bool is_q = j < nq;
      const int jj = is_q ? j : j - nq;
      const int s = jj % slots;
      act_t* dst = is_q ? q_out + ((size_t)t * nq + jj) * width
                        : k_pages + (((size_t)page * nkv + jj / slots) * TL_PAGE + in_page) * width;
      if (is_q && slots > 1) {
        for (int d = lane; d < width; d += 32)
          if (d < s * dim || d >= (s + 1) * dim) dst[d] = from_f32<act_t>(0.0f);
      }
#pragma unroll
      for (int r = 0; r < RA_MAX_DIM / 32; ++r) {
        const int d = lane + 32 * r;
        if (d < dim) dst[s * dim + d] = from_f32<act_t>(unit_norm ? keep[r] * inv : keep[r]);
      }
      __syncwarp();     // `mine` is rewritten by the warp's next vector
    } else {
      const int g = j - nq - nk;
      const float* src = row + (size_t)(nq + nk) * dim + (size_t)g * vdim;
      act_t* dst = v_pages + ((size_t)page * nv + g) * vdim * TL_PAGE + in_page;
      for (int d = lane; d < vdim; d += 32) dst[(size_t)d * TL_PAGE] = from_f32<act_t>(src[d]);
    }
  }
}

extern "C" int TL_NAME(tl_rotary_cache_write)(const float* z, int ldz, const float* inv_freq, int rot, int style,
                                              int unit_norm, float eps, void* q_out, void* k_pages, void* v_pages,
                                              const int* token_pos, const int* token_seq, const int* seq_slot,
                                              const int* page_table, int table_stride, int T, int nq, int nk,
                                              int nv, int dim, int vdim, int slots, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (nq < 1 || nk < 1 || nv < 1 || dim < 1 || vdim < 1 || slots < 1 || nq % slots || nk % slots ||
      nk / slots != nv || rot < 0 || rot > dim || (rot & 1) || (rot > 0 && inv_freq == nullptr))
    return TL_ERR_BAD_ARG;
  if (dim > RA_MAX_DIM) return TL_ERR_UNSUPPORTED;
  const int vectors = nq + nk + nv;
  const bool few = T < 512;
  const dim3 grid(T, few ? (vectors + RA_WARPS - 1) / RA_WARPS : 1);
  return tl_launch(rotary_cache_write_kernel, grid, dim3(RA_WARPS * 32), 0, stream, z, ldz, inv_freq, rot, style,
                   unit_norm, eps, (act_t*)q_out, (act_t*)k_pages, (act_t*)v_pages, token_pos, token_seq, seq_slot,
                   page_table, table_stride, nq, nk, nv, dim, vdim, slots);
}

// a: [T][heads][2][vdim] (the two maps' outputs of every head); out: [T][heads][vdim].
// o = a1 - lambda a2;  out = o / sqrt(mean(o^2) + eps) * mult.  A warp per (token, head).
#define DH_MAX_PER_LANE 16     // value sizes up to 512
__global__ void __launch_bounds__(256)
diff_heads_kernel(const act_t* __restrict__ a, float lambda, float eps, float mult, act_t* __restrict__ out,
                  int rows, int vdim) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const act_t* a1 = a + (size_t)r * 2 * vdim;
  const act_t* a2 = a1 + vdim;
  float o[DH_MAX_PER_LANE];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < DH_MAX_PER_LANE; ++i) {
    const int d = lane + 32 * i;
    o[i] = d < vdim ? to_f32(a1[d]) - lambda * to_f32(a2[d]) : 0.0f;
    ss = fmaf(o[i], o[i], ss);
  }
  ss = warp_sum(ss);
  const float f = mult / sqrtf(ss / (float)vdim + eps);
#pragma unroll
  for (int i = 0; i < DH_MAX_PER_LANE; ++i) {
    const int d = lane + 32 * i;
    if (d < vdim) out[(size_t)r * vdim + d] = from_f32<act_t>(o[i] * f);
  }
}

extern "C" int TL_NAME(tl_diff_heads)(const void* a, float lambda, float eps, float mult, void* out, int T,
                                      int heads, int vdim, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (heads < 1 || vdim < 1) return TL_ERR_BAD_ARG;
  if (vdim > 32 * DH_MAX_PER_LANE) return TL_ERR_UNSUPPORTED;
  const long long rows = (long long)T * heads;
  return tl_launch(diff_heads_kernel, dim3((unsigned)((rows + 7) / 8)), dim3(256), 0, stream, (const act_t*)a,
                   lambda, eps, mult, (act_t*)out, (int)rows, vdim);
}

// x[t, c] *= sigmoid(gate[t, c]); gate 32-bit with row stride ldg.
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(act_t* __restrict__ x, const float* __restrict__ gate, int ldg, int T, int n) {
  pdl_wait();
  pdl_launch_dependents();
  const long long total = (long long)T * n;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / n), c = (int)(i - (long long)t * n);
    const float g = 1.0f / (1.0f + expf(-gate[(size_t)t * ldg + c]));
    x[i] = from_f32<act_t>(to_f32(x[i]) * g);
  }
}

extern "C" int TL_NAME(tl_sigmoid_gate)(void* x, const float* gate, int ldg, int T, int n, cudaStream_t stream) {
  if (T <= 0 || n <= 0) return 0;
  const long long total = (long long)T * n;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  return tl_launch(sigmoid_gate_kernel, dim3(blocks), dim3(256), 0, stream, (act_t*)x, gate, ldg, T, n);
}
