// A short causal convolution over time, channel by channel, across the steps of a request, and
// what a layer with both sublayers on one norm needs around it.
//
//   short_conv        y[t, c] = f(sum_j w[c, j] * x[t - (taps - 1) + j, c] + bias[c]) (+ x[t, c] with
//                     `residual`), f the identity or silu; inputs before a request's first row of the
//                     step come from the taps - 1 inputs kept in its state slot (zeros at a
//                     sequence's start, because a slot starts zeroed).  A block a row.
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
                  const float* __restrict__ bias, const float* __restrict__ state, long long stride, int off,
                  const int* __restrict__ row_req, const int* __restrict__ q_start,
                  const int* __restrict__ state_slot, int act, int residual, TO* __restrict__ y) {
  const int t = blockIdx.x;
  const int r = row_req[t];
  pdl_wait();
  pdl_launch();
  if (r < 0) return;
  const int place = t - q_start[r];                   // the row's place in its request's portion
  const float* kept = taps > 1 ? state + (size_t)state_slot[r] * stride + off : nullptr;
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
                                   const float* bias, const float* state, long long stride, int off,
                                   const int* row_req, const int* q_start, const int* state_slot, int act,
                                   int residual, void* y, int y_dtype, int n_rows, cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (channels <= 0 || taps < 1 || taps > CONV_MAX_TAPS || (act != CONV_ACT_NONE && act != CONV_ACT_SILU) ||
      (taps > 1 && (state == nullptr || off < 0 || off + (long long)(taps - 1) * channels > stride)))
    return TOKB200_BAD_SIZE;
#define LAUNCH(TI, TO)                                                                                            \
  return launch_dependent(short_conv_kernel<TI, TO>, dim3(n_rows), dim3(256), 0, stream, (const TI*)x, ld, at,   \
                          channels, taps, w, bias, state, stride, off, row_req, q_start, state_slot, act,       \
                          residual, (TO*)y)
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

template <typename TA, typename TB>
static int scaled_add_norm_out(float* x, const void* a, int a_partials, long long a_stride, const float* va,
                               const void* b, int b_partials, long long b_stride, const float* vb, const float* gain,
                               float eps, void* y, int y_dtype, int n_rows, int hidden, cudaStream_t stream) {
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
