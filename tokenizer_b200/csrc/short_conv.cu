// A short causal convolution over time, channel by channel, across the steps of a request, and
// what a layer with both sublayers on one norm needs around it.
//
//   short_conv        y[t, c] = f(sum_j w[c, j] * x[t - (taps - 1) + j, c] + bias[c]) (+ x[t, c] with
//                     `residual`), f the identity or silu; inputs before a request's first row of the
//                     step come from the taps - 1 inputs kept in its state slot (zeros at a
//                     sequence's start, because a slot starts zeroed).  A block a row.  With `shift`
//                     (every request of the step brings ONE row) the row's block also moves the
//                     request's kept inputs on, which spares the launch below.
//   short_conv_state  the kept inputs move on by the step's rows (a thread a request and channel);
//                     launched behind short_conv, which reads the old ones.
//   scaled_add_norm   x += v1 * a (+ v2 * b), v float32 vectors over the width (a layer's learned
//                     scales), a and b sublayer outputs (bfloat16, float32, or float32 partial sums
//                     [S, T, H] added in index order); then, with a gain, y = x / sqrt(mean(x^2) +
//                     eps) * gain.  A block a row; sums in 32-bit.
//   embed_positions   x[t] = table[ids[t]] * scale + positions[pos[t]], 32-bit.
#include "common.cuh"

#define CONV_MAX_TAPS 16

enum : int { CONV_ACT_NONE = 0, CONV_ACT_SILU = 1 };

// x: [T, ld], the channels at columns `at` ..; state: [slots, stride] float32, a slot's kept inputs
// [taps - 1, channels] at `off` (kept[k] is the input taps - 1 - k rows before the next one).
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
short_conv_kernel(const TI* __restrict__ x, int ld, int at, int channels, int taps, const float* __restrict__ w,
                  const float* __restrict__ bias, float* state, long long stride, int off,
                  const int* __restrict__ row_req, const int* __restrict__ q_start,
                  const int* __restrict__ state_slot, int act, int residual, TO* __restrict__ y, int shift) {
  const int t = blockIdx.x;
  const int r = row_req[t];
  pdl_wait();
  pdl_launch();
  if (r < 0) return;
  const int place = t - q_start[r];                   // the row's place in its request's portion
  float* kept = taps > 1 ? state + (size_t)state_slot[r] * stride + off : nullptr;
  for (int c = threadIdx.x; c < channels; c += blockDim.x) {
    float acc = bias ? bias[c] : 0.f;
    float now = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;                  // tap j weighs the input `back` rows ago
      float v;
      if (back <= place) {
        v = to_float(x[(size_t)(t - back) * ld + at + c]);
      } else {
        v = kept[(size_t)(taps - 1 - (back - place)) * channels + c];
      }
      if (back == 0) now = v;
      acc = fmaf(w[(size_t)c * taps + j], v, acc);
    }
    if (act == CONV_ACT_SILU) acc = acc / (1.0f + expf(-acc));
    if (residual) acc += now;
    y[(size_t)t * channels + c] = from_float<TO>(acc);
    if (shift && taps > 1) {                          // the only row of its request: nobody else reads these
      for (int k = 0; k + 2 < taps; ++k) kept[(size_t)k * channels + c] = kept[(size_t)(k + 1) * channels + c];
      kept[(size_t)(taps - 2) * channels + c] = now;
    }
  }
}


// Four consecutive channels of a row (8 bytes of bfloat16, 16 of float32).
__device__ __forceinline__ float4 conv_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 conv_load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
  const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void conv_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void conv_store4(__nv_bfloat16* p, float4 v) {
  uint2 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
  h[0] = __floats2bfloat162_rn(v.x, v.y);
  h[1] = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = raw;
}

// Four channels as they lie in memory, unpacked only where they are used: a run's inputs wait in half the registers.
template <typename T> struct ConvRaw;
template <> struct ConvRaw<float> { typedef float4 type; };
template <> struct ConvRaw<__nv_bfloat16> { typedef uint2 type; };
__device__ __forceinline__ float4 conv_load_raw(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ uint2 conv_load_raw(const __nv_bfloat16* p) { return *reinterpret_cast<const uint2*>(p); }
__device__ __forceinline__ float4 conv_unpack(float4 v) { return v; }
__device__ __forceinline__ float4 conv_unpack(uint2 raw) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
  const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  return make_float4(a.x, a.y, b.x, b.y);
}

// The same convolution for 2 to 4 taps and channels in whole 4s: a thread owns four neighbouring channels.
// One row of it, wherever the row lies in its request's portion: the window is filled from the rows before it
// and, where the portion starts within TAPS - 1 rows, from the inputs kept in the request's slot.  Sums in the
// order of the kernel above.
template <int TAPS>
__device__ __forceinline__ float4 conv_row4(const float (&wt)[4][TAPS], const float4 (&win)[TAPS - 1], float4 now, float4 b4,
                                            int act, int residual) {
  float acc[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
  for (int k = 0; k < TAPS - 1; ++k) {
    acc[0] = fmaf(wt[0][k], win[k].x, acc[0]);
    acc[1] = fmaf(wt[1][k], win[k].y, acc[1]);
    acc[2] = fmaf(wt[2][k], win[k].z, acc[2]);
    acc[3] = fmaf(wt[3][k], win[k].w, acc[3]);
  }
  acc[0] = fmaf(wt[0][TAPS - 1], now.x, acc[0]);
  acc[1] = fmaf(wt[1][TAPS - 1], now.y, acc[1]);
  acc[2] = fmaf(wt[2][TAPS - 1], now.z, acc[2]);
  acc[3] = fmaf(wt[3][TAPS - 1], now.w, acc[3]);
  if (act == CONV_ACT_SILU) {
#pragma unroll
    for (int v = 0; v < 4; ++v) acc[v] = acc[v] / (1.0f + expf(-acc[v]));
  }
  if (residual) { acc[0] += now.x; acc[1] += now.y; acc[2] += now.z; acc[3] += now.w; }
  return make_float4(acc[0], acc[1], acc[2], acc[3]);
}

// A block covers ROWS consecutive rows of the step.  A run that lies inside one request's portion, at least
// TAPS - 1 rows behind its start, takes the straight path: the run's inputs and the TAPS - 1 rows in front of it
// are asked for at once, before anything is waited for, every input is loaded once and the window moves through
// registers.  Every other run (a portion's first rows, a border between requests, the step's last rows, a step
// of single tokens, which also moves the kept inputs on) goes row by row.
template <int TAPS, int ROWS, typename TI, typename TO>
__global__ void __launch_bounds__(128)
short_conv_tile_kernel(const TI* __restrict__ x, int ld, int at, int channels, const float* __restrict__ w,
                       const float* __restrict__ bias, float* state, long long stride, int off,
                       const int* __restrict__ row_req, const int* __restrict__ q_start,
                       const int* __restrict__ state_slot, int act, int residual, TO* __restrict__ y, int shift,
                       int n_rows) {
  typedef typename ConvRaw<TI>::type Raw;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  const int t0 = blockIdx.x * ROWS;
  pdl_wait();
  pdl_launch();
  if (c >= channels) return;
  float wt[4][TAPS];
  float4 win[TAPS - 1];                               // win[k]: the input TAPS - 1 - k rows before the current one
  if (ROWS > 1 && !shift && t0 >= TAPS - 1 && t0 + ROWS <= n_rows) {
    Raw in[ROWS], ahead[TAPS - 1];                    // ahead[k]: row t0 - (TAPS - 1 - k), whoever it belongs to
#pragma unroll
    for (int i = 0; i < ROWS; ++i) in[i] = conv_load_raw(x + (size_t)(t0 + i) * ld + at + c);
#pragma unroll
    for (int k = 0; k < TAPS - 1; ++k) ahead[k] = conv_load_raw(x + (size_t)(t0 - (TAPS - 1 - k)) * ld + at + c);
    const int r = row_req[t0];
    const int begin = r >= 0 ? q_start[r] : 0, end = r >= 0 ? q_start[r + 1] : 0;
    if (r >= 0 && begin + TAPS - 1 <= t0 && t0 + ROWS <= end) {
#pragma unroll
      for (int v = 0; v < 4; ++v)
#pragma unroll
        for (int j = 0; j < TAPS; ++j) wt[v][j] = w[(size_t)(c + v) * TAPS + j];
      const float4 b4 = bias ? *reinterpret_cast<const float4*>(bias + c) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int k = 0; k < TAPS - 1; ++k) win[k] = conv_unpack(ahead[k]);
#pragma unroll
      for (int i = 0; i < ROWS; ++i) {
        const float4 now = conv_unpack(in[i]);
        conv_store4(y + (size_t)(t0 + i) * channels + c, conv_row4<TAPS>(wt, win, now, b4, act, residual));
#pragma unroll
        for (int k = 0; k + 2 < TAPS; ++k) win[k] = win[k + 1];
        win[TAPS - 2] = now;
      }
      return;
    }
  }
#pragma unroll
  for (int v = 0; v < 4; ++v)
#pragma unroll
    for (int j = 0; j < TAPS; ++j) wt[v][j] = w[(size_t)(c + v) * TAPS + j];
  const float4 b4 = bias ? *reinterpret_cast<const float4*>(bias + c) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
  for (int t = t0; t < t0 + ROWS && t < n_rows; ++t) {
    const int r = row_req[t];
    if (r < 0) continue;
    const int place = t - q_start[r];
    float* kept = (place < TAPS - 1 || shift) ? state + (size_t)state_slot[r] * stride + off : nullptr;
#pragma unroll
    for (int k = 0; k < TAPS - 1; ++k) {
      const int back = TAPS - 1 - k;
      win[k] = back <= place ? conv_unpack(conv_load_raw(x + (size_t)(t - back) * ld + at + c))
                             : *reinterpret_cast<const float4*>(kept + (size_t)(TAPS - 1 - (back - place)) * channels + c);
    }
    const float4 now = conv_unpack(conv_load_raw(x + (size_t)t * ld + at + c));
    conv_store4(y + (size_t)t * channels + c, conv_row4<TAPS>(wt, win, now, b4, act, residual));
    if (shift) {                                      // the only row of its request: its kept inputs move on here
#pragma unroll
      for (int k = 0; k + 2 < TAPS; ++k) *reinterpret_cast<float4*>(kept + (size_t)k * channels + c) = win[k + 1];
      *reinterpret_cast<float4*>(kept + (size_t)(TAPS - 2) * channels + c) = now;
    }
  }
}

template <typename TI>
__global__ void short_conv_state_kernel(const TI* __restrict__ x, int ld, int at, int channels, int taps,
                                        float* __restrict__ state, long long stride, int off,
                                        const int* __restrict__ q_start, const int* __restrict__ state_slot) {
  const int r = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int first = q_start[r], n = q_start[r + 1] - first;
  pdl_wait();
  pdl_launch();
  if (n <= 0 || c >= channels) return;
  float* kept = state + (size_t)state_slot[r] * stride + off;
  // the last taps - 1 of (kept inputs, then the step's n inputs); ascending k reads kept[k + n]
  // before anything writes it
  for (int k = 0; k < taps - 1; ++k) {
    const int from = k + n;
    float v;
    if (from >= taps - 1) {
      v = to_float(x[(size_t)(first + from - (taps - 1)) * ld + at + c]);
    } else {
      v = kept[(size_t)from * channels + c];
    }
    kept[(size_t)k * channels + c] = v;
  }
}

TOKB200_API int tokb200_short_conv(const void* x, int x_dtype, int ld, int at, int channels, int taps, const float* w,
                                   const float* bias, float* state, long long stride, int off,
                                   const int* row_req, const int* q_start, const int* state_slot, int act,
                                   int residual, void* y, int y_dtype, int n_rows, int shift, cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (channels <= 0 || taps < 1 || taps > CONV_MAX_TAPS || (act != CONV_ACT_NONE && act != CONV_ACT_SILU) ||
      (taps > 1 && (state == nullptr || off < 0 || off + (long long)(taps - 1) * channels > stride)))
    return TOKB200_BAD_SIZE;
  const int x_size = x_dtype == TOKB200_BF16 ? 2 : 4, y_size = y_dtype == TOKB200_BF16 ? 2 : 4;
  if (taps >= 2 && taps <= 4 && channels % 4 == 0 && at % 4 == 0 && ld % 4 == 0 && off % 4 == 0 && stride % 4 == 0 &&
      ((uintptr_t)x % (4 * x_size)) == 0 && ((uintptr_t)y % (4 * y_size)) == 0 &&
      (((uintptr_t)state | (uintptr_t)bias) & 15) == 0) {
    // many rows: runs of 8 rows a thread; few (a decoding step): a row a thread, so that the blocks are many
    const int rows = n_rows >= 1024 ? 8 : 1;
    const int threads = channels / 4 >= 128 ? 128 : (channels / 4 + 31) / 32 * 32;
    const dim3 grid((n_rows + rows - 1) / rows, (channels / 4 + threads - 1) / threads);
#define TILE(TAPS, ROWS, TI, TO)                                                                                     \
    return launch_dependent(short_conv_tile_kernel<TAPS, ROWS, TI, TO>, grid, dim3(threads), 0, stream, (const TI*)x, \
                            ld, at, channels, w, bias, state, stride, off, row_req, q_start, state_slot, act,         \
                            residual, (TO*)y, shift, n_rows)
#define TILE_BY_TAPS(TI, TO)                                                    \
    if (taps == 2) { if (rows == 8) TILE(2, 8, TI, TO); TILE(2, 1, TI, TO); }   \
    if (taps == 3) { if (rows == 8) TILE(3, 8, TI, TO); TILE(3, 1, TI, TO); }   \
    if (rows == 8) TILE(4, 8, TI, TO);                                          \
    TILE(4, 1, TI, TO)
    if (grid.y <= 65535) {                  // the pairs of types that the layers use; the others take the kernel above
      if (x_dtype == TOKB200_F32 && y_dtype == TOKB200_F32) { TILE_BY_TAPS(float, float); }
      if (x_dtype == TOKB200_BF16 && y_dtype == TOKB200_BF16) { TILE_BY_TAPS(__nv_bfloat16, __nv_bfloat16); }
    }
#undef TILE_BY_TAPS
#undef TILE
  }
#define LAUNCH(TI, TO)                                                                                            \
  return launch_dependent(short_conv_kernel<TI, TO>, dim3(n_rows), dim3(256), 0, stream, (const TI*)x, ld, at,   \
                          channels, taps, w, bias, state, stride, off, row_req, q_start, state_slot, act,       \
                          residual, (TO*)y, shift)
  if (x_dtype == TOKB200_F32 && y_dtype == TOKB200_F32) LAUNCH(float, float);
  if (x_dtype == TOKB200_F32 && y_dtype == TOKB200_BF16) LAUNCH(float, __nv_bfloat16);
  if (x_dtype == TOKB200_BF16 && y_dtype == TOKB200_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  if (x_dtype == TOKB200_BF16 && y_dtype == TOKB200_F32) LAUNCH(__nv_bfloat16, float);
#undef LAUNCH
  return TOKB200_BAD_DTYPE;
}

TOKB200_API int tokb200_short_conv_state(const void* x, int x_dtype, int ld, int at, int channels, int taps,
                                         float* state, long long stride, int off, const int* q_start,
                                         const int* state_slot, int n_requests, cudaStream_t stream) {
  if (n_requests <= 0 || taps <= 1) return TOKB200_OK;
  if (channels <= 0 || taps > CONV_MAX_TAPS || off < 0 || off + (long long)(taps - 1) * channels > stride ||
      n_requests > 65535)
    return TOKB200_BAD_SIZE;
  const dim3 grid((channels + 127) / 128, n_requests);
  if (x_dtype == TOKB200_F32)
    return launch_dependent(short_conv_state_kernel<float>, grid, dim3(128), 0, stream, (const float*)x, ld, at,
                            channels, taps, state, stride, off, q_start, state_slot);
  if (x_dtype == TOKB200_BF16)
    return launch_dependent(short_conv_state_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream,
                            (const __nv_bfloat16*)x, ld, at, channels, taps, state, stride, off, q_start, state_slot);
  return TOKB200_BAD_DTYPE;
}

// ---- x += v1 * a + v2 * b, then the RMS norm of the new x --------------------------------------
#define SAN_MAX_PER_THREAD 8

template <typename T>
__device__ __forceinline__ float san_term(const T* __restrict__ y, int n_partials, size_t stride, size_t i) {
  float sum = to_float(y[i]);
  for (int s = 1; s < n_partials; ++s) sum += to_float(y[i + (size_t)s * stride]);
  return sum;
}

template <typename TA, typename TB, typename TO>
__global__ void __launch_bounds__(1024)
scaled_add_norm_kernel(float* __restrict__ x, const TA* __restrict__ a, int a_partials, size_t a_stride,
                       const float* __restrict__ va, const TB* __restrict__ b, int b_partials, size_t b_stride,
                       const float* __restrict__ vb, const float* __restrict__ gain, float eps, TO* __restrict__ y,
                       int hidden) {
  __shared__ float scratch[33];
  pdl_wait();
  pdl_launch();
  const size_t base = (size_t)blockIdx.x * hidden;
  float kept[SAN_MAX_PER_THREAD];
  float squares = 0.f;
#pragma unroll
  for (int k = 0; k < SAN_MAX_PER_THREAD; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    kept[k] = 0.f;
    if (i < hidden) {
      float v = x[base + i];
      v = fmaf(va[i], san_term(a, a_partials, a_stride, base + i), v);
      if (b != nullptr) v = fmaf(vb[i], san_term(b, b_partials, b_stride, base + i), v);
      x[base + i] = v;
      kept[k] = v;
      squares = fmaf(v, v, squares);
    }
  }
  for (int i = threadIdx.x + SAN_MAX_PER_THREAD * blockDim.x; i < hidden; i += blockDim.x) {   // rows wider than that
    float v = x[base + i];
    v = fmaf(va[i], san_term(a, a_partials, a_stride, base + i), v);
    if (b != nullptr) v = fmaf(vb[i], san_term(b, b_partials, b_stride, base + i), v);
    x[base + i] = v;
    squares = fmaf(v, v, squares);
  }
  if (gain == nullptr) return;
  const float total = block_sum(squares, scratch);
  const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
#pragma unroll
  for (int k = 0; k < SAN_MAX_PER_THREAD; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < hidden) y[base + i] = from_float<TO>(kept[k] * inv * gain[i]);
  }
  for (int i = threadIdx.x + SAN_MAX_PER_THREAD * blockDim.x; i < hidden; i += blockDim.x)
    y[base + i] = from_float<TO>(x[base + i] * inv * gain[i]);
}


__device__ __forceinline__ void store8(float* out, const float* v) {
  *reinterpret_cast<float4*>(out) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(out + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* out, const float* v) {
  uint4 packed;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
  for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
  *reinterpret_cast<uint4*>(out) = packed;
}

// Eight consecutive elements of a term (16 bytes of bfloat16; float32 planes added in index order).
__device__ __forceinline__ void san_load8(const __nv_bfloat16* __restrict__ y, int, size_t, size_t i, float* v) {
  const uint4 raw = *reinterpret_cast<const uint4*>(y + i);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = __bfloat1622float2(h[e]);
    v[2 * e] = f.x;
    v[2 * e + 1] = f.y;
  }
}
__device__ __forceinline__ void san_load8(const float* __restrict__ y, int n_partials, size_t stride, size_t i, float* v) {
#pragma unroll
  for (int e = 0; e < 8; ++e) v[e] = 0.f;
  for (int s = 0; s < n_partials; ++s) {
    const float4 lo = *reinterpret_cast<const float4*>(y + i + (size_t)s * stride);
    const float4 hi = *reinterpret_cast<const float4*>(y + i + (size_t)s * stride + 4);
    v[0] += lo.x; v[1] += lo.y; v[2] += lo.z; v[3] += lo.w; v[4] += hi.x; v[5] += hi.y; v[6] += hi.z; v[7] += hi.w;
  }
}

// Widths in whole 8s up to 8,192, everything 16-byte aligned: eight elements a thread with 16-byte loads,
// the row kept in registers between the sum and the scaling.
template <typename TA, typename TB, typename TO>
__global__ void __launch_bounds__(1024)
scaled_add_norm_rows_kernel(float* __restrict__ x, const TA* __restrict__ a, int a_partials, size_t a_stride,
                            const float* __restrict__ va, const TB* __restrict__ b, int b_partials, size_t b_stride,
                            const float* __restrict__ vb, const float* __restrict__ gain, float eps,
                            TO* __restrict__ y, int hidden) {
  __shared__ float scratch[33];
  pdl_wait();
  pdl_launch();
  const size_t base = (size_t)blockIdx.x * hidden;
  const int c = threadIdx.x * 8;
  const bool on = c < hidden;
  float v[8];
  float squares = 0.f;
  if (on) {
    const float4 x0 = *reinterpret_cast<const float4*>(x + base + c);
    const float4 x1 = *reinterpret_cast<const float4*>(x + base + c + 4);
    v[0] = x0.x; v[1] = x0.y; v[2] = x0.z; v[3] = x0.w; v[4] = x1.x; v[5] = x1.y; v[6] = x1.z; v[7] = x1.w;
    float t[8], s[8];
    san_load8(a, a_partials, a_stride, base + c, t);
    *reinterpret_cast<float4*>(s) = *reinterpret_cast<const float4*>(va + c);
    *reinterpret_cast<float4*>(s + 4) = *reinterpret_cast<const float4*>(va + c + 4);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = fmaf(s[e], t[e], v[e]);
    if (b != nullptr) {
      san_load8(b, b_partials, b_stride, base + c, t);
      *reinterpret_cast<float4*>(s) = *reinterpret_cast<const float4*>(vb + c);
      *reinterpret_cast<float4*>(s + 4) = *reinterpret_cast<const float4*>(vb + c + 4);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = fmaf(s[e], t[e], v[e]);
    }
    *reinterpret_cast<float4*>(x + base + c) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(x + base + c + 4) = make_float4(v[4], v[5], v[6], v[7]);
#pragma unroll
    for (int e = 0; e < 8; ++e) squares = fmaf(v[e], v[e], squares);
  }
  if (gain == nullptr) return;
  const float inv = 1.0f / sqrtf(block_sum(squares, scratch) / (float)hidden + eps);
  if (on) {
    float g[8];
    *reinterpret_cast<float4*>(g) = *reinterpret_cast<const float4*>(gain + c);
    *reinterpret_cast<float4*>(g + 4) = *reinterpret_cast<const float4*>(gain + c + 4);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = v[e] * inv * g[e];
    store8(y + base + c, v);
  }
}

template <typename TA, typename TB>
static int scaled_add_norm_out(float* x, const void* a, int a_partials, long long a_stride, const float* va,
                               const void* b, int b_partials, long long b_stride, const float* vb, const float* gain,
                               float eps, void* y, int y_dtype, int n_rows, int hidden, cudaStream_t stream) {
  const int y_size = y_dtype == TOKB200_BF16 ? 2 : 4;
  if (hidden % 8 == 0 && hidden <= 8192 && a_stride % 4 == 0 && b_stride % 4 == 0 &&
      (((uintptr_t)x | (uintptr_t)a | (uintptr_t)b | (uintptr_t)va | (uintptr_t)vb | (uintptr_t)gain | (uintptr_t)y) & 15) == 0 &&
      ((size_t)hidden * sizeof(TA)) % 16 == 0 && ((size_t)hidden * sizeof(TB)) % 16 == 0 && ((size_t)hidden * y_size) % 16 == 0) {
    const int threads8 = (hidden / 8 + 31) / 32 * 32;
#define LAUNCH8(TO)                                                                                               \
    return launch_dependent(scaled_add_norm_rows_kernel<TA, TB, TO>, dim3(n_rows), dim3(threads8), 0, stream, x,  \
                            (const TA*)a, a_partials, (size_t)a_stride, va, (const TB*)b, b_partials,             \
                            (size_t)b_stride, vb, gain, eps, (TO*)y, hidden)
    if (y_dtype == TOKB200_BF16) LAUNCH8(__nv_bfloat16);
    LAUNCH8(float);
#undef LAUNCH8
  }
  int threads = ((hidden + 3) / 4 + 31) / 32 * 32;
  threads = threads < 32 ? 32 : threads > 1024 ? 1024 : threads;
#define LAUNCH(TO)                                                                                              \
  return launch_dependent(scaled_add_norm_kernel<TA, TB, TO>, dim3(n_rows), dim3(threads), 0, stream, x,        \
                          (const TA*)a, a_partials, (size_t)a_stride, va, (const TB*)b, b_partials,             \
                          (size_t)b_stride, vb, gain, eps, (TO*)y, hidden)
  if (y_dtype == TOKB200_BF16) LAUNCH(__nv_bfloat16);
  LAUNCH(float);
#undef LAUNCH
}

// a, b: [T, H] of their dtype or float32 partial sums (n > 1, `stride` elements apart); b may be null.
// gain null: the add alone.
TOKB200_API int tokb200_scaled_add_norm(float* x, const void* a, int a_dtype, int a_partials, long long a_stride,
                                        const float* va, const void* b, int b_dtype, int b_partials,
                                        long long b_stride, const float* vb, const float* gain, float eps, void* y,
                                        int y_dtype, int n_rows, int hidden, cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (hidden <= 0 || a == nullptr || va == nullptr || (b != nullptr && vb == nullptr) || a_partials < 1 ||
      b_partials < 1 || (gain != nullptr && y == nullptr))
    return TOKB200_BAD_SIZE;
  if ((a_partials > 1 && a_dtype != TOKB200_F32) || (b_partials > 1 && b_dtype != TOKB200_F32)) return TOKB200_BAD_DTYPE;
#define GO(TA, TB)                                                                                                  \
  return scaled_add_norm_out<TA, TB>(x, a, a_partials, a_stride, va, b, b_partials, b_stride, vb, gain, eps, y,     \
                                     y_dtype, n_rows, hidden, stream)
  const int bt = b == nullptr ? a_dtype : b_dtype;
  if (a_dtype == TOKB200_F32 && bt == TOKB200_F32) GO(float, float);
  if (a_dtype == TOKB200_F32 && bt == TOKB200_BF16) GO(float, __nv_bfloat16);
  if (a_dtype == TOKB200_BF16 && bt == TOKB200_F32) GO(__nv_bfloat16, float);
  if (a_dtype == TOKB200_BF16 && bt == TOKB200_BF16) GO(__nv_bfloat16, __nv_bfloat16);
#undef GO
  return TOKB200_BAD_DTYPE;
}

// ---- token embedding plus a learned vector of the token's position ----------------------------
template <typename T>
__global__ void embed_positions_kernel(const int* __restrict__ ids, const int* __restrict__ pos,
                                       const int* __restrict__ row_req, const T* __restrict__ table,
                                       const T* __restrict__ positions, float* __restrict__ x, int hidden, int vocab,
                                       int n_positions, float scale) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x;
  int id = ids[t];
  int p = pos[t];
  if (id < 0 || id >= vocab) id = 0;              // ids and lengths are validated on the host; never read outside
  if (p < 0 || p >= n_positions || row_req[t] < 0) p = 0;
  const T* row = table + (size_t)id * hidden;
  const T* prow = positions + (size_t)p * hidden;
  float* out = x + (size_t)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = fmaf(to_float(row[i]), scale, to_float(prow[i]));
}

TOKB200_API int tokb200_embed_positions(const int* ids, const int* pos, const int* row_req, const void* table,
                                        const void* positions, int dtype, float* x, int n_tokens, int hidden,
                                        int vocab, int n_positions, float scale, cudaStream_t stream) {
  if (n_tokens <= 0) return TOKB200_OK;
  if (hidden <= 0 || vocab <= 0 || n_positions <= 0) return TOKB200_BAD_SIZE;
  if (dtype == TOKB200_F32)
    return launch_dependent(embed_positions_kernel<float>, dim3(n_tokens), dim3(256), 0, stream, ids, pos, row_req,
                            (const float*)table, (const float*)positions, x, hidden, vocab, n_positions, scale);
  if (dtype == TOKB200_BF16)
    return launch_dependent(embed_positions_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), 0, stream, ids, pos,
                            row_req, (const __nv_bfloat16*)table, (const __nv_bfloat16*)positions, x, hidden, vocab,
                            n_positions, scale);
  return TOKB200_BAD_DTYPE;
}
