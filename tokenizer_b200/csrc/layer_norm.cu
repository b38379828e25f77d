// Layer norm with gain and bias, y = (x - mean) / sqrt(var + eps) * gain + bias (var: the mean of
// the squared deviations, taken in a second pass over the row), and the residual stream's steps
// of a layer that norms its sublayers' outputs as well as their inputs:
//
//   layer_norm          out = LN(x) (optionally of gathered rows)
//   post_norm_add       x += LN_post(y);  optionally out = LN_next(x): the norm on a sublayer's output,
//                       the residual add and the norm in front of the next sublayer in one pass
//                       (`rms` / `next_rms`: that norm is the RMS form instead, y / sqrt(mean(y^2) + eps) * gain,
//                       with a bias only where one is given)
//   scaled_sum          out = s1 y1 + s2 y2
//   stream_inject       x += other + vector: what a pass of a looped stack adds before its first layer
//
// y is a sum of up to two scaled terms (two mixers side by side), each [T, H] in float32 or
// bfloat16 or float32 partial sums [S, T, H] of a product cut along k, added in index order.
// One block a row; a thread keeps up to LN_PER_THREAD elements in registers between the passes
// (wider rows are read again).  Statistics and the stream are 32-bit.
#include "common.cuh"

#define LN_PER_THREAD 8

struct LnTerm {
  const void* y;       // null: no term
  int bf16;            // the term's elements are bfloat16 (else float32)
  int n_partials;
  long long stride;    // elements between partial sums
  float scale;
};

__device__ __forceinline__ float ln_term(const LnTerm& t, size_t at) {
  if (t.y == nullptr) return 0.f;
  float v = 0.f;
  if (t.bf16) {
    v = __bfloat162float(((const __nv_bfloat16*)t.y)[at]);
  } else {
    const float* y = (const float*)t.y;
    for (int s = 0; s < t.n_partials; ++s) v += y[(size_t)s * t.stride + at];
  }
  return v * t.scale;
}

// mean and 1 / sqrt(var + eps) of the row's n values, which the caller hands over through `get`
template <typename F>
__device__ __forceinline__ void ln_statistics(F get, int n, float eps, float* scratch, float& mean, float& inv,
                                              int rms = 0) {
  float s = 0.f;
  if (!rms)
    for (int i = threadIdx.x; i < n; i += blockDim.x) s += get(i);
  mean = rms ? 0.f : block_sum(s, scratch) / (float)n;      // the RMS form takes no mean off
  float q = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float d = get(i) - mean;
    q += d * d;
  }
  inv = 1.0f / sqrtf(block_sum(q, scratch) / (float)n + eps);
}

template <typename TO>
__global__ void __launch_bounds__(1024)
layer_norm_kernel(const float* __restrict__ x, const float* __restrict__ gain, const float* __restrict__ bias,
                  TO* __restrict__ out, const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_wait();
  pdl_launch();
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * hidden;
  TO* o = out + (size_t)r * hidden;
  const bool kept = hidden <= LN_PER_THREAD * (int)blockDim.x;
  float v[LN_PER_THREAD];
#pragma unroll
  for (int e = 0; e < LN_PER_THREAD; ++e) {
    const int i = threadIdx.x + e * blockDim.x;
    v[e] = (kept && i < hidden) ? xr[i] : 0.f;
  }
  float mean, inv;
  if (kept) {
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < LN_PER_THREAD; ++e) s += v[e];
    mean = block_sum(s, scratch) / (float)hidden;
    float q = 0.f;
#pragma unroll
    for (int e = 0; e < LN_PER_THREAD; ++e) {
      const int i = threadIdx.x + e * blockDim.x;
      const float d = i < hidden ? v[e] - mean : 0.f;
      q += d * d;
    }
    inv = 1.0f / sqrtf(block_sum(q, scratch) / (float)hidden + eps);
#pragma unroll
    for (int e = 0; e < LN_PER_THREAD; ++e) {
      const int i = threadIdx.x + e * blockDim.x;
      if (i < hidden) o[i] = from_float<TO>((v[e] - mean) * inv * gain[i] + bias[i]);
    }
  } else {
    ln_statistics([&](int i) { return xr[i]; }, hidden, eps, scratch, mean, inv);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
      o[i] = from_float<TO>((xr[i] - mean) * inv * gain[i] + bias[i]);
  }
}

template <typename TO>
__global__ void __launch_bounds__(1024)
post_norm_add_kernel(float* __restrict__ x, LnTerm t1, LnTerm t2, const float* __restrict__ gain,
                     const float* __restrict__ bias, float eps, const float* __restrict__ next_gain,
                     const float* __restrict__ next_bias, float next_eps, TO* __restrict__ out, int hidden,
                     int rms, int next_rms) {
  __shared__ float scratch[33];
  pdl_wait();
  pdl_launch();
  const int r = blockIdx.x;
  const size_t base = (size_t)r * hidden;
  float* xr = x + base;
  const bool kept = hidden <= LN_PER_THREAD * (int)blockDim.x;
  if (kept) {
    float v[LN_PER_THREAD], xv[LN_PER_THREAD];
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < LN_PER_THREAD; ++e) {
      const int i = threadIdx.x + e * blockDim.x;
      v[e] = i < hidden ? ln_term(t1, base + i) + ln_term(t2, base + i) : 0.f;
      xv[e] = i < hidden ? xr[i] : 0.f;
      s += v[e];
    }
    const float mean = rms ? 0.f : block_sum(s, scratch) / (float)hidden;
    float q = 0.f;
#pragma unroll
    for (int e = 0; e < LN_PER_THREAD; ++e) {
      const int i = threadIdx.x + e * blockDim.x;
      const float d = i < hidden ? v[e] - mean : 0.f;
      q += d * d;
    }
    const float inv = 1.0f / sqrtf(block_sum(q, scratch) / (float)hidden + eps);
    s = 0.f;
#pragma unroll
    for (int e = 0; e < LN_PER_THREAD; ++e) {
      const int i = threadIdx.x + e * blockDim.x;
      if (i < hidden) {
        xv[e] += (v[e] - mean) * inv * gain[i] + (bias ? bias[i] : 0.f);
        xr[i] = xv[e];
        s += xv[e];
      }
    }
    if (out == nullptr) return;
    const float mean2 = next_rms ? 0.f : block_sum(s, scratch) / (float)hidden;
    q = 0.f;
#pragma unroll
    for (int e = 0; e < LN_PER_THREAD; ++e) {
      const int i = threadIdx.x + e * blockDim.x;
      const float d = i < hidden ? xv[e] - mean2 : 0.f;
      q += d * d;
    }
    const float inv2 = 1.0f / sqrtf(block_sum(q, scratch) / (float)hidden + next_eps);
    TO* o = out + base;
#pragma unroll
    for (int e = 0; e < LN_PER_THREAD; ++e) {
      const int i = threadIdx.x + e * blockDim.x;
      if (i < hidden) o[i] = from_float<TO>((xv[e] - mean2) * inv2 * next_gain[i] + (next_bias ? next_bias[i] : 0.f));
    }
    return;
  }
  float mean, inv;
  ln_statistics([&](int i) { return ln_term(t1, base + i) + ln_term(t2, base + i); }, hidden, eps, scratch, mean, inv, rms);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    xr[i] += (ln_term(t1, base + i) + ln_term(t2, base + i) - mean) * inv * gain[i] + (bias ? bias[i] : 0.f);
  if (out == nullptr) return;
  __syncthreads();
  ln_statistics([&](int i) { return xr[i]; }, hidden, next_eps, scratch, mean, inv, next_rms);
  TO* o = out + base;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    o[i] = from_float<TO>((xr[i] - mean) * inv * next_gain[i] + (next_bias ? next_bias[i] : 0.f));
}

// ---- rows whose width is whole 8s: eight consecutive elements a thread, 16-byte loads ----
__device__ __forceinline__ void ln_load8(const float* p, float v[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

__device__ __forceinline__ void ln_store8(float* p, const float v[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

__device__ __forceinline__ void ln_store8(__nv_bfloat16* p, const float v[8]) {
  __nv_bfloat162 h[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(h);
}

// adds the term's eight elements at `at`, scaled, to v
__device__ __forceinline__ void ln_term8(const LnTerm& t, size_t at, float v[8]) {
  if (t.y == nullptr) return;
  if (t.bf16) {
    const uint4 raw = *reinterpret_cast<const uint4*>((const __nv_bfloat16*)t.y + at);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      v[2 * i] += f.x * t.scale;
      v[2 * i + 1] += f.y * t.scale;
    }
    return;
  }
  float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < t.n_partials; ++s) {
    float part[8];
    ln_load8((const float*)t.y + (size_t)s * t.stride + at, part);
#pragma unroll
    for (int i = 0; i < 8; ++i) sum[i] += part[i];
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] += sum[i] * t.scale;
}

template <typename TO>
__global__ void __launch_bounds__(1024)
post_norm_add_rows8_kernel(float* __restrict__ x, LnTerm t1, LnTerm t2, const float* __restrict__ gain,
                           const float* __restrict__ bias, float eps, const float* __restrict__ next_gain,
                           const float* __restrict__ next_bias, float next_eps, TO* __restrict__ out, int hidden,
                           int rms, int next_rms) {
  __shared__ float scratch[33];
  // gains and biases are weights: asked for before the wait on the predecessor
  const int i0 = threadIdx.x * 8;
  const bool on = i0 < hidden;
  float g[8], b[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (on) {
    ln_load8(gain + i0, g);
    if (bias) ln_load8(bias + i0, b);
  }
  pdl_wait();
  pdl_launch();
  const size_t base = (size_t)blockIdx.x * hidden + i0;
  float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, xv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (on) {
    ln_load8(x + base, xv);
    ln_term8(t1, base, v);
    ln_term8(t2, base, v);
  }
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) s += v[i];
  const float mean = rms ? 0.f : block_sum(s, scratch) / (float)hidden;
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) q += on ? (v[i] - mean) * (v[i] - mean) : 0.f;
  const float inv = 1.0f / sqrtf(block_sum(q, scratch) / (float)hidden + eps);
  s = 0.f;
  if (on) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      xv[i] += (v[i] - mean) * inv * g[i] + b[i];
      s += xv[i];
    }
    ln_store8(x + base, xv);
  }
  if (out == nullptr) return;
  if (on) {
    ln_load8(next_gain + i0, g);
    if (next_bias) ln_load8(next_bias + i0, b);
    else {
#pragma unroll
      for (int i = 0; i < 8; ++i) b[i] = 0.f;
    }
  }
  const float mean2 = next_rms ? 0.f : block_sum(s, scratch) / (float)hidden;
  q = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) q += on ? (xv[i] - mean2) * (xv[i] - mean2) : 0.f;
  const float inv2 = 1.0f / sqrtf(block_sum(q, scratch) / (float)hidden + next_eps);
  if (on) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = (xv[i] - mean2) * inv2 * g[i] + b[i];
    ln_store8(out + base, v);
  }
}

__global__ void scaled_sum_kernel(LnTerm t1, LnTerm t2, float* __restrict__ out, size_t n) {
  pdl_wait();
  pdl_launch();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = ln_term(t1, i) + ln_term(t2, i);
}

// x[t, :] += other[t, :] (where given) + vector[:] (where given)
__global__ void stream_inject_kernel(float* __restrict__ x, const float* __restrict__ other,
                                     const float* __restrict__ vector, int hidden, size_t n) {
  pdl_wait();
  pdl_launch();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    x[i] += (other ? other[i] : 0.f) + (vector ? vector[i % hidden] : 0.f);
}

static inline int ln_threads(int hidden) {
  int threads = 128;   // rows of up to 4 elements a thread at first, 8 in the widest block
  while (threads < 1024 && hidden > threads * 4) threads *= 2;
  return threads;
}

static inline LnTerm ln_make_term(const void* y, int dtype, int n_partials, long long stride, float scale) {
  LnTerm t;
  t.y = y;
  t.bf16 = dtype == TOKB200_BF16;
  t.n_partials = n_partials;
  t.stride = stride;
  t.scale = scale;
  return t;
}

TOKB200_API int tokb200_layer_norm(const float* x, const float* gain, const float* bias, void* out, int out_dtype,
                                   const int* rows, int n_rows, int hidden, float eps, cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (hidden <= 0) return TOKB200_BAD_SIZE;
  const int threads = ln_threads(hidden);
  if (out_dtype == TOKB200_F32)
    return launch_dependent(layer_norm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, gain, bias,
                            (float*)out, rows, hidden, eps);
  if (out_dtype == TOKB200_BF16)
    return launch_dependent(layer_norm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, x, gain,
                            bias, (__nv_bfloat16*)out, rows, hidden, eps);
  return TOKB200_BAD_DTYPE;
}

// y2 may be null (one term).  out may be null (no norm behind the add).
TOKB200_API int tokb200_post_norm_add(float* x, const void* y1, int y1_dtype, int y1_partials, long long y1_stride,
                                      float y1_scale, const void* y2, int y2_dtype, int y2_partials,
                                      long long y2_stride, float y2_scale, const float* gain, const float* bias,
                                      float eps, const float* next_gain, const float* next_bias, float next_eps,
                                      void* out, int out_dtype, int n_rows, int hidden, int rms, int next_rms,
                                      cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (hidden <= 0 || y1 == nullptr || y1_partials < 1 || (y2 && y2_partials < 1)) return TOKB200_BAD_SIZE;
  if ((!rms && bias == nullptr) || (out != nullptr && !next_rms && next_bias == nullptr)) return TOKB200_BAD_SIZE;
  if ((y1_dtype == TOKB200_BF16 && y1_partials != 1) || (y2 && y2_dtype == TOKB200_BF16 && y2_partials != 1))
    return TOKB200_BAD_DTYPE;
  const LnTerm t1 = ln_make_term(y1, y1_dtype, y1_partials, y1_stride, y1_scale);
  const LnTerm t2 = ln_make_term(y2, y2_dtype, y2_partials, y2_stride, y2_scale);
  // whole 8s of up to 8,192 elements, everything on 16 bytes: eight elements a thread
  const uintptr_t all = (uintptr_t)x | (uintptr_t)y1 | (uintptr_t)y2 | (uintptr_t)gain | (uintptr_t)bias |
                        (uintptr_t)next_gain | (uintptr_t)next_bias | (uintptr_t)out;
  if (hidden % 8 == 0 && hidden <= 8192 && (all & 15) == 0 && y1_stride % 4 == 0 && y2_stride % 4 == 0) {
    const int threads8 = ((hidden / 8 + 31) / 32) * 32;
    if (out == nullptr || out_dtype == TOKB200_F32)
      return launch_dependent(post_norm_add_rows8_kernel<float>, dim3(n_rows), dim3(threads8), 0, stream, x, t1, t2,
                              gain, bias, eps, next_gain, next_bias, next_eps, (float*)out, hidden, rms, next_rms);
    if (out_dtype == TOKB200_BF16)
      return launch_dependent(post_norm_add_rows8_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads8), 0, stream, x,
                              t1, t2, gain, bias, eps, next_gain, next_bias, next_eps, (__nv_bfloat16*)out, hidden,
                              rms, next_rms);
    return TOKB200_BAD_DTYPE;
  }
  const int threads = ln_threads(hidden);
  if (out == nullptr || out_dtype == TOKB200_F32)
    return launch_dependent(post_norm_add_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, t1, t2, gain,
                            bias, eps, next_gain, next_bias, next_eps, (float*)out, hidden, rms, next_rms);
  if (out_dtype == TOKB200_BF16)
    return launch_dependent(post_norm_add_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, x, t1, t2,
                            gain, bias, eps, next_gain, next_bias, next_eps, (__nv_bfloat16*)out, hidden, rms,
                            next_rms);
  return TOKB200_BAD_DTYPE;
}

TOKB200_API int tokb200_scaled_sum(const void* y1, int y1_dtype, int y1_partials, long long y1_stride, float y1_scale,
                                   const void* y2, int y2_dtype, int y2_partials, long long y2_stride,
                                   float y2_scale, float* out, long long n, cudaStream_t stream) {
  if (n <= 0) return TOKB200_OK;
  if (y1 == nullptr || y1_partials < 1 || (y2 && y2_partials < 1)) return TOKB200_BAD_SIZE;
  const LnTerm t1 = ln_make_term(y1, y1_dtype, y1_partials, y1_stride, y1_scale);
  const LnTerm t2 = ln_make_term(y2, y2_dtype, y2_partials, y2_stride, y2_scale);
  const long long blocks = (n + 255) / 256;
  return launch_dependent(scaled_sum_kernel, dim3((unsigned)(blocks < 4096 ? blocks : 4096)), dim3(256), 0, stream,
                          t1, t2, out, (size_t)n);
}

TOKB200_API int tokb200_stream_inject(float* x, const float* other, const float* vector, int n_rows, int hidden,
                                      cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (hidden <= 0) return TOKB200_BAD_SIZE;
  const long long n = (long long)n_rows * hidden, blocks = (n + 255) / 256;
  return launch_dependent(stream_inject_kernel, dim3((unsigned)(blocks < 4096 ? blocks : 4096)), dim3(256), 0, stream,
                          x, other, vector, hidden, (size_t)n);
}
