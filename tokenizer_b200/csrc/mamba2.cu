// The selective state-space recurrence with a scalar decay a head (the Mamba-2 form), in 32-bit.
//
// Per head a matrix S (N x P, float32, a request's state) and per token t of that head:
//     dt = softplus(raw_dt + dt_bias);  S <- exp(-exp(A_log) dt) S + dt B x^T;  y = S^T C + D x
// with x (P lanes of the head), B and C (N lanes of the head's group) the convolved and activated
// inputs.  The columns of S are independent (column p needs x_p only), so thread (column p, part j)
// keeps the rows j, j + 8, j + 16, ... of column p in registers; the 8 parts of a column add their
// shares of S^T C in one round of shuffles.
//
//   mamba2_scan      the recurrence over every request's rows of the step, token by token; tokens are
//                    staged through shared memory in runs.  Grid: (blocks of 32 columns, heads,
//                    requests).  State: [slots, stride], a slot's matrices [heads, P, N] at its start.
//   mamba2_out_norm  y * silu(z), divided by its root mean square inside each of `parts` equal parts
//                    of the row, times a gain: a block a (row, part).
#include "common.cuh"

#define M2_PARTS 8                 // threads that share a column
#define M2_COLS 32                 // columns a block
#define M2_THREADS (M2_PARTS * M2_COLS)
#define M2_RUN 16                  // tokens staged at a time

__device__ __forceinline__ float m2_softplus(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// xbc: float32 [T, channels]: x (heads * P), B (groups * N), C (groups * N).  proj: the input product
// [T, ld] whose columns dt_at .. + heads are the raw step sizes.
template <int NPER, typename TI>
__global__ void __launch_bounds__(M2_THREADS)
mamba2_scan_kernel(const float* __restrict__ xbc, int channels, const TI* __restrict__ proj, int ld, int dt_at,
                   const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ skip,
                   int heads, int groups, int P, int N, float* __restrict__ state, long long stride,
                   const int* __restrict__ q_start, const int* __restrict__ state_slot, float* __restrict__ y) {
  constexpr int NPAD = NPER * M2_PARTS;
  __shared__ float Bs[M2_RUN][NPAD];
  __shared__ float Cs[M2_RUN][NPAD];
  __shared__ float xs[M2_RUN][M2_COLS];
  __shared__ float dts[M2_RUN];
  __shared__ float decs[M2_RUN];
  const int head = blockIdx.y, r = blockIdx.z;
  const int col0 = blockIdx.x * M2_COLS;
  const int part = threadIdx.x % M2_PARTS, col = col0 + threadIdx.x / M2_PARTS;
  const int group = head / (heads / groups);
  const int inner = heads * P;
  const float a = expf(a_log[head]), bias = dt_bias[head], d = skip[head];
  pdl_wait();
  pdl_launch();
  const int first = q_start[r], n = q_start[r + 1] - first;
  if (n <= 0) return;
  float* mine = state + (size_t)state_slot[r] * stride + ((size_t)head * P + col) * N;
  float S[NPER];
#pragma unroll
  for (int i = 0; i < NPER; ++i) {
    const int row = i * M2_PARTS + part;
    S[i] = (col < P && row < N) ? mine[row] : 0.f;
  }
  for (int run = 0; run < n; run += M2_RUN) {
    const int here = n - run < M2_RUN ? n - run : M2_RUN;
    __syncthreads();                       // the run before is read to its end
    for (int i = threadIdx.x; i < here * NPAD; i += M2_THREADS) {
      const int k = i / NPAD, row = i % NPAD;
      const float* src = xbc + (size_t)(first + run + k) * channels + inner + group * N;
      Bs[k][row] = row < N ? src[row] : 0.f;
      Cs[k][row] = row < N ? src[(size_t)groups * N + row] : 0.f;
    }
    for (int i = threadIdx.x; i < here * M2_COLS; i += M2_THREADS) {
      const int k = i / M2_COLS, c = col0 + i % M2_COLS;
      xs[k][i % M2_COLS] = c < P ? xbc[(size_t)(first + run + k) * channels + head * P + c] : 0.f;
    }
    if (threadIdx.x < here) {
      const float dt = m2_softplus(to_float(proj[(size_t)(first + run + threadIdx.x) * ld + dt_at + head]) + bias);
      dts[threadIdx.x] = dt;
      decs[threadIdx.x] = expf(-a * dt);
    }
    __syncthreads();
    for (int k = 0; k < here; ++k) {
      const float x = xs[k][threadIdx.x / M2_PARTS];
      const float dec = decs[k], dtx = dts[k] * x;
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < NPER; ++i) {
        const int row = i * M2_PARTS + part;
        S[i] = fmaf(dec, S[i], dtx * Bs[k][row]);
        acc = fmaf(S[i], Cs[k][row], acc);
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      if (part == 0 && col < P) y[(size_t)(first + run + k) * inner + head * P + col] = fmaf(d, x, acc);
    }
  }
#pragma unroll
  for (int i = 0; i < NPER; ++i) {
    const int row = i * M2_PARTS + part;
    if (col < P && row < N) mine[row] = S[i];
  }
}

TOKB200_API int tokb200_mamba2_scan(const float* xbc, int channels, const void* proj, int proj_dtype, int ld, int dt_at,
                                    const float* dt_bias, const float* a_log, const float* skip, int heads, int groups,
                                    int P, int N, float* state, long long stride, const int* q_start,
                                    const int* state_slot, int n_requests, float* y, cudaStream_t stream) {
  if (n_requests <= 0) return TOKB200_OK;
  if (heads <= 0 || groups <= 0 || heads % groups || P <= 0 || N <= 0 || N > 32 * M2_PARTS || heads > 65535 ||
      n_requests > 65535 || channels != heads * P + 2 * groups * N || (long long)heads * P * N > stride)
    return TOKB200_BAD_SIZE;
  const dim3 grid((P + M2_COLS - 1) / M2_COLS, heads, n_requests);
#define LAUNCH(NPER, TI)                                                                                          \
  return launch_dependent(mamba2_scan_kernel<NPER, TI>, grid, dim3(M2_THREADS), 0, stream, xbc, channels,          \
                          (const TI*)proj, ld, dt_at, dt_bias, a_log, skip, heads, groups, P, N, state, stride,     \
                          q_start, state_slot, y)
#define BY_SIZE(TI)                                   \
  if (N <= 4 * M2_PARTS) LAUNCH(4, TI);               \
  if (N <= 8 * M2_PARTS) LAUNCH(8, TI);               \
  if (N <= 16 * M2_PARTS) LAUNCH(16, TI);             \
  LAUNCH(32, TI)
  if (proj_dtype == TOKB200_F32) { BY_SIZE(float); }
  if (proj_dtype == TOKB200_BF16) { BY_SIZE(__nv_bfloat16); }
#undef BY_SIZE
#undef LAUNCH
  return TOKB200_BAD_DTYPE;
}

// y: float32 [T, inner]; z: the gate's pre-activation, columns z_at .. + inner of `proj` [T, ld].
#define M2_NORM_PER_THREAD 8
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
mamba2_out_norm_kernel(const float* __restrict__ y, const TI* __restrict__ proj, int ld, int z_at,
                       const float* __restrict__ gain, float eps, int inner, int parts,
                       const int* __restrict__ row_req, TO* __restrict__ out) {
  __shared__ float scratch[33];
  const int t = blockIdx.x, g = blockIdx.y;
  const int width = inner / parts;
  pdl_wait();
  pdl_launch();
  if (row_req[t] < 0) return;
  const float* yr = y + (size_t)t * inner + (size_t)g * width;
  const TI* zr = proj + (size_t)t * ld + z_at + (size_t)g * width;
  float kept[M2_NORM_PER_THREAD];
  float squares = 0.f;
#pragma unroll
  for (int k = 0; k < M2_NORM_PER_THREAD; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    kept[k] = 0.f;
    if (i < width) {
      const float z = to_float(zr[i]);
      const float v = yr[i] * (z / (1.0f + expf(-z)));
      kept[k] = v;
      squares = fmaf(v, v, squares);
    }
  }
  for (int i = threadIdx.x + M2_NORM_PER_THREAD * blockDim.x; i < width; i += blockDim.x) {
    const float z = to_float(zr[i]);
    const float v = yr[i] * (z / (1.0f + expf(-z)));
    squares = fmaf(v, v, squares);
  }
  const float inv = 1.0f / sqrtf(block_sum(squares, scratch) / (float)width + eps);
  TO* o = out + (size_t)t * inner + (size_t)g * width;
  const float* gr = gain + (size_t)g * width;
#pragma unroll
  for (int k = 0; k < M2_NORM_PER_THREAD; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < width) o[i] = from_float<TO>(kept[k] * inv * gr[i]);
  }
  for (int i = threadIdx.x + M2_NORM_PER_THREAD * blockDim.x; i < width; i += blockDim.x) {
    const float z = to_float(zr[i]);
    o[i] = from_float<TO>(yr[i] * (z / (1.0f + expf(-z))) * inv * gr[i]);
  }
}

TOKB200_API int tokb200_mamba2_out_norm(const float* y, const void* proj, int proj_dtype, int ld, int z_at,
                                        const float* gain, float eps, int inner, int parts, const int* row_req,
                                        void* out, int out_dtype, int n_rows, cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (inner <= 0 || parts <= 0 || inner % parts || parts > 65535) return TOKB200_BAD_SIZE;
  const int width = inner / parts;
  int threads = (width + 31) / 32 * 32;
  threads = threads > 256 ? 256 : threads;
  const dim3 grid(n_rows, parts);
#define LAUNCH(TI, TO)                                                                                           \
  return launch_dependent(mamba2_out_norm_kernel<TI, TO>, grid, dim3(threads), 0, stream, y, (const TI*)proj, ld, \
                          z_at, gain, eps, inner, parts, row_req, (TO*)out)
  if (proj_dtype == TOKB200_F32 && out_dtype == TOKB200_F32) LAUNCH(float, float);
  if (proj_dtype == TOKB200_F32 && out_dtype == TOKB200_BF16) LAUNCH(float, __nv_bfloat16);
  if (proj_dtype == TOKB200_BF16 && out_dtype == TOKB200_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  if (proj_dtype == TOKB200_BF16 && out_dtype == TOKB200_F32) LAUNCH(__nv_bfloat16, float);
#undef LAUNCH
  return TOKB200_BAD_DTYPE;
}
