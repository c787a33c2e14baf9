// Kernels of a block that norms every sublayer's input and output,
//     x <- x + N_out(sublayer(N_in(x))),        N(u) = u / sqrt(mean(u^2) + eps) * w,
// and two activations of feed-forwards.
//
//   norm_add_norm   x += N_out(y) in the 32-bit stream, and, if the next norm's weight is given,
//                   xn = N_next(x) in the activation type in the same pass: the stream crosses
//                   memory once per sublayer.
//   relu_squared    out = max(z, 0)^2.
//   clamped_glu     z = [g | u] per row: g <- min(g, limit), u <- clamp(u, -limit, limit),
//                   out = g * sigmoid(alpha g) * (u + 1).
#include "common.cuh"

#define SW_KEEP 8

// One block per row.  y: [rows, H] 32-bit with row stride ldy; w_out, w_next: norm weights in their
// stored type (32-bit or bfloat16, `w32` says which).
__global__ void norm_add_norm_kernel(const float* __restrict__ y, int ldy, const void* __restrict__ w_out,
                                     const void* __restrict__ w_next, int w32, float eps_out, float eps_next,
                                     float* __restrict__ x, act_t* __restrict__ xn, int H) {
  __shared__ float scratch[33];
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const float* yr = y + (size_t)r * ldy;
  float* xr = x + (size_t)r * H;
  const bool fits = H <= (int)blockDim.x * SW_KEEP;
  auto weight = [&](const void* w, int i) {
    return w32 ? ((const float*)w)[i] : __bfloat162float(((const __nv_bfloat16*)w)[i]);
  };
  float keep[SW_KEEP], xs[SW_KEEP], wo[SW_KEEP];
  float ss = 0.0f;
  if (fits) {
    // the stream and the weight are asked for before the first sum, so that they arrive during it
#pragma unroll
    for (int j = 0; j < SW_KEEP; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      keep[j] = i < H ? yr[i] : 0.0f;
      xs[j] = i < H ? xr[i] : 0.0f;
      wo[j] = i < H ? weight(w_out, i) : 0.0f;
      ss = fmaf(keep[j], keep[j], ss);
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) ss = fmaf(yr[i], yr[i], ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps_out);
  float s2 = 0.0f;
  if (fits) {
#pragma unroll
    for (int j = 0; j < SW_KEEP; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < H) {
        const float v = xs[j] + keep[j] * inv * wo[j];
        xr[i] = v;
        keep[j] = v;
        s2 = fmaf(v, v, s2);
      }
    }
    if (w_next != nullptr) {
#pragma unroll
      for (int j = 0; j < SW_KEEP; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        wo[j] = i < H ? weight(w_next, i) : 0.0f;
      }
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      const float v = xr[i] + yr[i] * inv * weight(w_out, i);
      xr[i] = v;
      s2 = fmaf(v, v, s2);
    }
  }
  if (w_next == nullptr) return;
  s2 = block_sum(s2, scratch);
  const float inv2 = 1.0f / sqrtf(s2 / (float)H + eps_next);
  act_t* o = xn + (size_t)r * H;
  if (fits) {
#pragma unroll
    for (int j = 0; j < SW_KEEP; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < H) o[i] = from_f32<act_t>(keep[j] * inv2 * wo[j]);
    }
  } else {
    // every thread reads back what it wrote itself
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<act_t>(xr[i] * inv2 * weight(w_next, i));
  }
}

extern "C" int TL_NAME(tl_norm_add_norm)(const float* y, int ldy, const void* w_out, const void* w_next, int w32,
                                         float eps_out, float eps_next, float* x, void* xn, int rows, int H,
                                         cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H <= 0 || w_out == nullptr || (w_next != nullptr && xn == nullptr)) return TL_ERR_BAD_ARG;
  const int threads = H <= 1024 ? 128 : H <= 2048 ? 256 : 512;
  return tl_launch(norm_add_norm_kernel, dim3(rows), dim3(threads), 0, stream, y, ldy, w_out, w_next, w32, eps_out,
                   eps_next, x, (act_t*)xn, H);
}

__global__ void __launch_bounds__(256)
relu_squared_kernel(const float* __restrict__ z, int ldz, act_t* __restrict__ out, int T, int n) {
  pdl_wait();
  pdl_launch_dependents();
  const long long total = (long long)T * n;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / n), c = (int)(i - (long long)t * n);
    const float v = fmaxf(z[(size_t)t * ldz + c], 0.0f);
    out[i] = from_f32<act_t>(v * v);
  }
}

extern "C" int TL_NAME(tl_relu_squared)(const float* z, int ldz, void* out, int T, int n, cudaStream_t stream) {
  if (T <= 0 || n <= 0) return 0;
  const long long total = (long long)T * n;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  return tl_launch(relu_squared_kernel, dim3(blocks), dim3(256), 0, stream, z, ldz, (act_t*)out, T, n);
}

__global__ void __launch_bounds__(256)
clamped_glu_kernel(const float* __restrict__ z, int ldz, float limit, float alpha, act_t* __restrict__ out, int T,
                   int n) {
  pdl_wait();
  pdl_launch_dependents();
  const long long total = (long long)T * n;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / n), c = (int)(i - (long long)t * n);
    const float g = fminf(z[(size_t)t * ldz + c], limit);
    const float u = fminf(fmaxf(z[(size_t)t * ldz + n + c], -limit), limit);
    out[i] = from_f32<act_t>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
  }
}

extern "C" int TL_NAME(tl_clamped_glu)(const float* z, int ldz, float limit, float alpha, void* out, int T, int n,
                                       cudaStream_t stream) {
  if (T <= 0 || n <= 0) return 0;
  const long long total = (long long)T * n;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  return tl_launch(clamped_glu_kernel, dim3(blocks), dim3(256), 0, stream, z, ldz, limit, alpha, (act_t*)out, T, n);
}
