// What stands around the paged attention kernels for mixers whose queries and keys are rotated
// by position: the step's projections on their way into the cache, and two ways of closing a
// head's output (the difference of two attention maps; a gate per output entry).
//
//   rotary_cache_write   z (32-bit rows: query vectors, key vectors, value heads side by side)
//                        -> rotated (and, if asked, unit-normed) q in the activation type, rotated
//                        k and plain v into the token's place in the pages.  `bias` (one number per
//                        column of z, or null) is added as the columns are read; the value heads
//                        start at column `v_col`, which may be where the key vectors start (the
//                        values are then the keys as projected, before rotation and norm).
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
rotary_cache_write_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ bias, int v_col,
                          const float* __restrict__ inv_freq, int rot,
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
      const float* bj = bias != nullptr ? bias + (size_t)j * dim : nullptr;
      for (int d = lane; d < dim; d += 32) mine[d] = src[d] + (bj != nullptr ? bj[d] : 0.0f);
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
      const size_t col = (size_t)v_col + (size_t)g * vdim;
      const float* src = row + col;
      act_t* dst = v_pages + ((size_t)page * nv + g) * vdim * TL_PAGE + in_page;
      for (int d = lane; d < vdim; d += 32)
        dst[(size_t)d * TL_PAGE] = from_f32<act_t>(src[d] + (bias != nullptr ? bias[col + d] : 0.0f));
    }
  }
}

// Four values at a time.
__device__ __forceinline__ void ra_load4(const float* p, float (&v)[4]) {
  const float4 f = *reinterpret_cast<const float4*>(p);
  v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
}
__device__ __forceinline__ void ra_load4(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void ra_store4(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void ra_store4(__nv_bfloat16* p, const float (&v)[4]) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 u;
  u.x = *reinterpret_cast<const uint32_t*>(&a);
  u.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

// Four columns of a row of projections from column `at` on, with the columns' bias if there is one.
__device__ __forceinline__ void ra_load4_biased(const float* row, const float* bias, size_t at, float (&v)[4]) {
  ra_load4(row + at, v);
  if (bias != nullptr) {
    float b[4];
    ra_load4(bias + at, b);
#pragma unroll
    for (int e = 0; e < 4; ++e) v[e] += b[e];
  }
}

// The same for steps of many tokens.  Two kinds of block in one launch:
//  - blockIdx.x < T: one token.  The cosines and sines of its position are computed once (one per
//    rotated pair) into shared memory; then a warp per query or key vector, the warp's next vector
//    already on its way from memory while it works on this one;
//  - the blocks after them: 32 consecutive tokens of one value head each; the tile is turned in
//    shared memory, so that the transposed value pages are written in runs of positions.
// R: 32-entry pieces of a vector per lane (dim <= 32 R).
#define RAM_WARPS 8
template <int R>
__global__ void __launch_bounds__(RAM_WARPS * 32)
rotary_cache_write_many_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ bias, int v_col,
                               const float* __restrict__ inv_freq, int rot,
                               int style, int unit_norm, float eps, act_t* __restrict__ q_out,
                               act_t* __restrict__ k_pages, act_t* __restrict__ v_pages,
                               const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                               const int* __restrict__ seq_slot, const int* __restrict__ page_table,
                               int table_stride, int T, int nq, int nk, int nv, int dim, int vdim, int slots) {
  extern __shared__ float ra_sm[];
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if ((int)blockIdx.x >= T) {
    // ---- a tile of values: [32 tokens][vdim + 1] in shared memory
    const int tile = blockIdx.x - T;
    const int t0 = (tile / nv) * 32, g = tile % nv;
    const int nt = min(32, T - t0);
    const size_t col = (size_t)v_col + (size_t)g * vdim;
    const float* src = z + col;
    for (int idx = threadIdx.x; idx < nt * vdim; idx += blockDim.x) {
      const int tt = idx / vdim, d = idx - tt * vdim;
      ra_sm[tt * (vdim + 1) + d] = src[(size_t)(t0 + tt) * ldz + d] + (bias != nullptr ? bias[col + d] : 0.0f);
    }
    __syncthreads();
    if (lane < nt) {
      const int t = t0 + lane;
      const int pos = token_pos[t];
      const int page = page_table[(size_t)seq_slot[token_seq[t]] * table_stride + pos / TL_PAGE];
      act_t* dst = v_pages + ((size_t)page * nv + g) * vdim * TL_PAGE + (pos % TL_PAGE);
      for (int d = warp; d < vdim; d += RAM_WARPS) dst[(size_t)d * TL_PAGE] = from_f32<act_t>(ra_sm[lane * (vdim + 1) + d]);
    }
    return;
  }
  // ---- a token's query and key vectors
  const int t = blockIdx.x;
  const int pos = token_pos[t];
  const int slot = seq_slot[token_seq[t]];
  const int page = page_table[(size_t)slot * table_stride + pos / TL_PAGE];
  const int in_page = pos % TL_PAGE;
  const float* row = z + (size_t)t * ldz;
  const int half = rot / 2;
  const int width = slots * dim;
  const int nkv = nk / slots;
  float2* cs = reinterpret_cast<float2*>(ra_sm);            // [half] (cosine, sine)
  float* mine = ra_sm + 2 * half + warp * dim;             // [RAM_WARPS][dim]
  const float fpos = (float)pos;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, c;
    sincosf(fpos * inv_freq[i], &sn, &c);
    cs[i] = make_float2(c, sn);
  }
  __syncthreads();
  float cur[R], nxt[R];
  int j = warp;
  if (j < nq + nk) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int d = lane + 32 * r;
      cur[r] = d < dim ? row[(size_t)j * dim + d] + (bias != nullptr ? bias[(size_t)j * dim + d] : 0.0f) : 0.0f;
    }
  }
  for (; j < nq + nk; j += RAM_WARPS) {
    const int jn = j + RAM_WARPS;
    if (jn < nq + nk) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int d = lane + 32 * r;
        nxt[r] = d < dim ? row[(size_t)jn * dim + d] + (bias != nullptr ? bias[(size_t)jn * dim + d] : 0.0f) : 0.0f;
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int d = lane + 32 * r;
      if (d < rot) mine[d] = cur[r];
    }
    __syncwarp();
    float ss = 0.0f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int d = lane + 32 * r;
      float v = cur[r];
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
        const float2 c = cs[i];
        const float o = mine[partner];
        // (u, v) -> (u cos - v sin, v cos + u sin)
        v = first ? v * c.x - o * c.y : v * c.x + o * c.y;
      }
      cur[r] = v;
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
    for (int r = 0; r < R; ++r) {
      const int d = lane + 32 * r;
      if (d < dim) dst[s * dim + d] = from_f32<act_t>(unit_norm ? cur[r] * inv : cur[r]);
    }
    __syncwarp();     // `mine` is rewritten by the warp's next vector
#pragma unroll
    for (int r = 0; r < R; ++r) cur[r] = nxt[r];
  }
}

// The many-token kernel for vectors of 16, 32, 64 or 128 entries: a lane holds four neighbouring entries
// (16-byte loads, 8- or 16-byte stores), LPV lanes a vector, so a warp works on 32 / LPV vectors at a
// time.  The partner of a rotation lies in the same lane (pairs (2i, 2i + 1)) or rot/8 lanes away
// (pairs (i, i + rot/2); rot a multiple of 8), so nothing is staged in shared memory but the sines.
template <int LPV>
__global__ void __launch_bounds__(RAM_WARPS * 32)
rotary_cache_write_vec_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ bias, int v_col,
                              const float* __restrict__ inv_freq, int rot,
                              int style, int unit_norm, float eps, act_t* __restrict__ q_out,
                              act_t* __restrict__ k_pages, act_t* __restrict__ v_pages,
                              const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                              const int* __restrict__ seq_slot, const int* __restrict__ page_table,
                              int table_stride, int T, int nq, int nk, int nv, int vdim, int slots) {
  extern __shared__ float ra_sm[];
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int dim = 4 * LPV, VPW = 32 / LPV;
  if ((int)blockIdx.x >= T) {
    // ---- a tile of values: [32 tokens][vdim + 1] in shared memory
    const int tile = blockIdx.x - T;
    const int t0 = (tile / nv) * 32, g = tile % nv;
    const int nt = min(32, T - t0);
    const size_t col = (size_t)v_col + (size_t)g * vdim;
    const float* src = z + col;
    for (int idx = threadIdx.x; idx < nt * vdim; idx += blockDim.x) {
      const int tt = idx / vdim, d = idx - tt * vdim;
      ra_sm[tt * (vdim + 1) + d] = src[(size_t)(t0 + tt) * ldz + d] + (bias != nullptr ? bias[col + d] : 0.0f);
    }
    __syncthreads();
    if (lane < nt) {
      const int t = t0 + lane;
      const int pos = token_pos[t];
      const int page = page_table[(size_t)seq_slot[token_seq[t]] * table_stride + pos / TL_PAGE];
      act_t* dst = v_pages + ((size_t)page * nv + g) * vdim * TL_PAGE + (pos % TL_PAGE);
      for (int d = warp; d < vdim; d += RAM_WARPS) dst[(size_t)d * TL_PAGE] = from_f32<act_t>(ra_sm[lane * (vdim + 1) + d]);
    }
    return;
  }
  const int t = blockIdx.x;
  const int pos = token_pos[t];
  const float* row = z + (size_t)t * ldz;
  const int half = rot / 2;
  const int total = nq + nk;
  const int sub = lane / LPV, l = lane % LPV, d0 = 4 * l;
  // the first vectors are on their way while the sines are computed
  int j = warp * VPW + sub;
  float v[4] = {0.0f, 0.0f, 0.0f, 0.0f}, nx[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  if (j < total) ra_load4_biased(row, bias, (size_t)j * dim + d0, v);
  float2* cs = reinterpret_cast<float2*>(ra_sm);            // [half] (cosine, sine)
  const float fpos = (float)pos;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, c;
    sincosf(fpos * inv_freq[i], &sn, &c);
    cs[i] = make_float2(c, sn);
  }
  const int slot = seq_slot[token_seq[t]];
  const int page = page_table[(size_t)slot * table_stride + pos / TL_PAGE];
  const int in_page = pos % TL_PAGE;
  const int width = slots * dim;
  const int nkv = nk / slots;
  const int hl = half >> 2;                                  // lanes between the partners (pairs (i, i + half))
  const int partner = (lane - l) + (l < hl ? l + hl : (l < 2 * hl ? l - hl : l));
  __syncthreads();
  for (int j0 = warp * VPW; j0 < total; j0 += RAM_WARPS * VPW) {
    j = j0 + sub;
    const int jn = j + RAM_WARPS * VPW;
    if (jn < total) ra_load4_biased(row, bias, (size_t)jn * dim + d0, nx);
    float o[4];
    if (style == 0) {
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = __shfl_sync(0xffffffffu, v[e], partner);
    } else {
      o[0] = v[1]; o[1] = v[0]; o[2] = v[3]; o[3] = v[2];
    }
    float ss = 0.0f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int d = d0 + e;
      if (d < rot) {
        const bool first = style == 0 ? d < half : (e & 1) == 0;
        const int i = style == 0 ? (first ? d : d - half) : d >> 1;
        const float2 c = cs[i];
        // (u, v) -> (u cos - v sin, v cos + u sin)
        v[e] = first ? v[e] * c.x - o[e] * c.y : v[e] * c.x + o[e] * c.y;
      }
      ss = fmaf(v[e], v[e], ss);
    }
    if (unit_norm) {
#pragma unroll
      for (int m = LPV / 2; m > 0; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
      const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] *= inv;
    }
    if (j < total) {
      const bool is_q = j < nq;
      const int jj = is_q ? j : j - nq;
      const int s = jj % slots;
      act_t* dst = is_q ? q_out + ((size_t)t * nq + jj) * width
                        : k_pages + (((size_t)page * nkv + jj / slots) * TL_PAGE + in_page) * width;
      if (is_q && slots > 1) {
        const float zero[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int other = 0; other < slots; ++other)
          if (other != s) ra_store4(dst + other * dim + d0, zero);
      }
      ra_store4(dst + s * dim + d0, v);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) v[e] = nx[e];
  }
}

extern "C" int TL_NAME(tl_rotary_cache_write)(const float* z, int ldz, const float* bias, int v_col,
                                              const float* inv_freq, int rot, int style,
                                              int unit_norm, float eps, void* q_out, void* k_pages, void* v_pages,
                                              const int* token_pos, const int* token_seq, const int* seq_slot,
                                              const int* page_table, int table_stride, int T, int nq, int nk,
                                              int nv, int dim, int vdim, int slots, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (nq < 1 || nk < 1 || nv < 1 || dim < 1 || vdim < 1 || slots < 1 || nq % slots || nk % slots ||
      nk / slots != nv || rot < 0 || rot > dim || (rot & 1) || (rot > 0 && inv_freq == nullptr) || v_col < 0)
    return TL_ERR_BAD_ARG;
  if (dim > RA_MAX_DIM) return TL_ERR_UNSUPPORTED;
  const int vectors = nq + nk + nv;
  const size_t tile_bytes = (size_t)32 * (vdim + 1) * sizeof(float);
  const size_t token_bytes = (size_t)(rot + RAM_WARPS * dim) * sizeof(float);
  const size_t smem = tile_bytes > token_bytes ? tile_bytes : token_bytes;
  if (T >= 256 && smem <= 48 * 1024) {
    const unsigned blocks = (unsigned)T + (unsigned)((T + 31) / 32) * (unsigned)nv;
    const bool quads = (dim == 16 || dim == 32 || dim == 64 || dim == 128) && ldz % 4 == 0 && ((uintptr_t)z & 15) == 0 &&
                       ((uintptr_t)q_out & 15) == 0 && ((uintptr_t)k_pages & 15) == 0 && (style != 0 || rot % 8 == 0) &&
                       ((uintptr_t)bias & 15) == 0;
    if (quads) {
#define RA_VEC(LPV_)                                                                                                \
      return tl_launch(rotary_cache_write_vec_kernel<LPV_>, dim3(blocks), dim3(RAM_WARPS * 32), smem, stream, z,   \
                       ldz, bias, v_col, inv_freq, rot, style, unit_norm, eps, (act_t*)q_out, (act_t*)k_pages, (act_t*)v_pages, \
                       token_pos, token_seq, seq_slot, page_table, table_stride, T, nq, nk, nv, vdim, slots)
      if (dim == 16) RA_VEC(4);
      if (dim == 32) RA_VEC(8);
      if (dim == 64) RA_VEC(16);
      RA_VEC(32);
#undef RA_VEC
    }
#define RA_MANY(R_)                                                                                                  \
    return tl_launch(rotary_cache_write_many_kernel<R_>, dim3(blocks), dim3(RAM_WARPS * 32), smem, stream, z, ldz,  \
                     bias, v_col, inv_freq, rot, style, unit_norm, eps, (act_t*)q_out, (act_t*)k_pages, (act_t*)v_pages,         \
                     token_pos, token_seq, seq_slot, page_table, table_stride, T, nq, nk, nv, dim, vdim, slots)
    if (dim <= 32) RA_MANY(1);
    if (dim <= 64) RA_MANY(2);
    if (dim <= 128) RA_MANY(4);
    RA_MANY(8);
#undef RA_MANY
  }
  const dim3 grid(T, (vectors + RA_WARPS - 1) / RA_WARPS);
  return tl_launch(rotary_cache_write_kernel, grid, dim3(RA_WARPS * 32), 0, stream, z, ldz, bias, v_col, inv_freq, rot, style,
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

// The same with four values per lane at a time (value sizes that are multiples of 4, up to 512).
template <int N>     // 128-entry pieces of a head's values per warp (vdim <= 128 N)
__global__ void __launch_bounds__(256)
diff_heads_vec_kernel(const act_t* __restrict__ a, float lambda, float eps, float mult, act_t* __restrict__ out,
                      int rows, int vdim) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const act_t* a1 = a + (size_t)r * 2 * vdim;
  const act_t* a2 = a1 + vdim;
  float o[N][4];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < N; ++i) {
    const int d = (lane + 32 * i) * 4;
    float x[4] = {0.0f, 0.0f, 0.0f, 0.0f}, y[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (d < vdim) { ra_load4(a1 + d, x); ra_load4(a2 + d, y); }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      o[i][e] = x[e] - lambda * y[e];
      ss = fmaf(o[i][e], o[i][e], ss);
    }
  }
  ss = warp_sum(ss);
  const float f = mult / sqrtf(ss / (float)vdim + eps);
#pragma unroll
  for (int i = 0; i < N; ++i) {
    const int d = (lane + 32 * i) * 4;
    if (d < vdim) {
      float w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) w[e] = o[i][e] * f;
      ra_store4(out + (size_t)r * vdim + d, w);
    }
  }
}

extern "C" int TL_NAME(tl_diff_heads)(const void* a, float lambda, float eps, float mult, void* out, int T,
                                      int heads, int vdim, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (heads < 1 || vdim < 1) return TL_ERR_BAD_ARG;
  if (vdim > 32 * DH_MAX_PER_LANE) return TL_ERR_UNSUPPORTED;
  const long long rows = (long long)T * heads;
  if (vdim % 4 == 0 && vdim <= 512 && ((uintptr_t)a & 15) == 0 && ((uintptr_t)out & 15) == 0) {
#define DH_VEC(N_)                                                                                                \
    return tl_launch(diff_heads_vec_kernel<N_>, dim3((unsigned)((rows + 7) / 8)), dim3(256), 0, stream,          \
                     (const act_t*)a, lambda, eps, mult, (act_t*)out, (int)rows, vdim)
    if (vdim <= 128) DH_VEC(1);
    if (vdim <= 256) DH_VEC(2);
    DH_VEC(4);
#undef DH_VEC
  }
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

// The same, four entries per thread (n and ldg multiples of 4, 16-byte aligned rows).
__global__ void __launch_bounds__(256)
sigmoid_gate_vec_kernel(act_t* __restrict__ x, const float* __restrict__ gate, int ldg, int T, int n4) {
  pdl_wait();
  pdl_launch_dependents();
  const long long total = (long long)T * n4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / n4), c = (int)(i - (long long)t * n4) * 4;
    float g[4], v[4];
    ra_load4(gate + (size_t)t * ldg + c, g);
    act_t* p = x + (size_t)t * n4 * 4 + c;
    ra_load4(p, v);
#pragma unroll
    for (int e = 0; e < 4; ++e) v[e] = v[e] / (1.0f + expf(-g[e]));
    ra_store4(p, v);
  }
}

extern "C" int TL_NAME(tl_sigmoid_gate)(void* x, const float* gate, int ldg, int T, int n, cudaStream_t stream) {
  if (T <= 0 || n <= 0) return 0;
  if (n % 4 == 0 && ldg % 4 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)gate & 15) == 0) {
    const long long quads = (long long)T * (n / 4);
    const int vb = (int)((quads + 255) / 256 < 148 * 16 ? (quads + 255) / 256 : 148 * 16);
    return tl_launch(sigmoid_gate_vec_kernel, dim3(vb), dim3(256), 0, stream, (act_t*)x, gate, ldg, T, n / 4);
  }
  const long long total = (long long)T * n;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  return tl_launch(sigmoid_gate_kernel, dim3(blocks), dim3(256), 0, stream, (act_t*)x, gate, ldg, T, n);
}
