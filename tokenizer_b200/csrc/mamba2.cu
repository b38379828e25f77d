// The selective state-space recurrence with a scalar decay a head (the Mamba-2 form), in 32-bit.
//
// Per head a matrix S (N x P, float32, a request's state) and per token t of that head:
//     dt = softplus(raw_dt + dt_bias);  S <- exp(-exp(A_log) dt) S + dt B x^T;  y = S^T C + D x
// with x (P lanes of the head), B and C (N lanes of the head's group) the convolved and activated
// inputs.  The columns of S are independent (column p needs x_p only), so a thread keeps NPER neighbouring
// rows (rows j NPER .. (j + 1) NPER - 1 for part j) of TWO neighbouring columns in registers and reads a
// token's B and C once for both; the 8 parts of a column add their shares of S^T C by shuffles, eight
// tokens in 4 + 2 + 1 exchanges.  The rows' arithmetic is packed: two rows an instruction.
//
//   mamba2_scan      the recurrence over every request's rows of the step, token by token.  Tokens are
//                    staged through shared memory in runs (cp.async, the next run on its way while
//                    the current one is computed); a part's rows of B and C lie side by side there,
//                    padded so that the 16-byte reads of the 8 parts fall on different banks.  Grid:
//                    (blocks of 32 columns, heads, requests).  State: [slots, stride], a slot's
//                    matrices [heads, P, N] at its start.
//   mamba2_out_norm  y * silu(z), divided by its root mean square inside each of `parts` equal parts
//                    of the row, times a gain: a block a (row, part).
#include "common.cuh"

#define M2_PARTS 8                 // threads that share a column
#define M2_COLS 32                 // columns a block
#define M2_OWN 2                   // neighbouring columns a thread: B and C are read once for both
#define M2_THREADS (M2_PARTS * M2_COLS / M2_OWN)

__device__ __forceinline__ float m2_softplus(float v) { return v > 20.f ? v : log1pf(expf(v)); }

__device__ __forceinline__ void m2_copy4(float* dst, const float* src) {
  const unsigned to = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(to), "l"(src) : "memory");
}

__device__ __forceinline__ void m2_copy16(float* dst, const float* src) {
  const unsigned to = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(to), "l"(src) : "memory");
}

// xbc: float32 [T, channels]: x (heads * P), B (groups * N), C (groups * N).  proj: the input product
// [T, ld] whose columns dt_at .. + heads are the raw step sizes.
//
// PASS 0 runs a request's rows from first to last.  PASS 1 and 2 together do the same with a request's rows cut
// into up to `segments` equal segments (whole 16s of rows) that run side by side, for steps whose requests are
// too few to fill the device: the recurrence is linear in S, so a segment's end is (product of its decays) *
// (its start) + (its end from a zero start).  PASS 1: segment 0 runs in full from the slot's matrices; every
// other segment but the last runs from zero without reading C or writing y and leaves its end and the product
// of its decays in `scratch`.  PASS 2: every segment from the second on folds the ends before it into its start,
// then runs in full; the last one writes the slot.  (A request with one segment is done in PASS 1.)
// scratch: [requests, segments, heads, P, N] ends, then [requests, segments, heads] products.
template <int NPER, typename TI, int PASS>
__global__ void __launch_bounds__(M2_THREADS)
mamba2_scan_kernel(const float* __restrict__ xbc, int channels, const TI* __restrict__ proj, int ld, int dt_at,
                   const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ skip,
                   int heads, int groups, int P, int N, float* __restrict__ state, long long stride,
                   const int* __restrict__ q_start, const int* __restrict__ state_slot, float* __restrict__ y,
                   float* __restrict__ scratch, int segments, int n_requests) {
  constexpr int RUN = NPER >= 32 ? 8 : 16;            // tokens staged at a time
  constexpr int PADDED = NPER + 4;                    // a part's rows and four idle lanes
  constexpr int NPAD = PADDED * M2_PARTS;
  __shared__ __align__(16) float Bs[2][RUN][NPAD];
  __shared__ __align__(16) float Cs[2][RUN][NPAD];
  __shared__ __align__(16) float xs[2][RUN][M2_COLS];
  __shared__ float dts[2][RUN];
  __shared__ float decs[2][RUN];
  const int head = blockIdx.y, r = PASS == 0 ? blockIdx.z : blockIdx.z / segments;
  const int seg = PASS == 0 ? 0 : blockIdx.z % segments;
  const int col0 = blockIdx.x * M2_COLS;
  const int part = threadIdx.x % M2_PARTS, mine_x = (threadIdx.x / M2_PARTS) * M2_OWN, col = col0 + mine_x;
  const int group = head / (heads / groups);
  const int inner = heads * P;
  const float a = expf(a_log[head]), bias = dt_bias[head], d = skip[head];
  // lanes that no copy reaches (rows from N on, columns from P on) stay zero in both halves
  if (N < NPER * M2_PARTS) {
    for (int i = threadIdx.x; i < 2 * RUN * NPAD; i += M2_THREADS) {
      (&Bs[0][0][0])[i] = 0.f;
      (&Cs[0][0][0])[i] = 0.f;
    }
  }
  if (P - col0 < M2_COLS)
    for (int i = threadIdx.x; i < 2 * RUN * M2_COLS; i += M2_THREADS) (&xs[0][0][0])[i] = 0.f;
  pdl_wait();
  pdl_launch();
  int first = q_start[r], n = q_start[r + 1] - first;
  if (n <= 0) return;
  float* mine = state + (size_t)state_slot[r] * stride + ((size_t)head * P + col) * N;
  float2 S[M2_OWN][NPER / 2];              // pairs of neighbouring rows: the arithmetic below is packed, two lanes an instruction
  // a thread's rows are neighbours in the slot: 16-byte loads where the matrix has whole runs of them
  const bool whole = N == NPER * M2_PARTS && col + M2_OWN <= P && (stride & 3) == 0 && ((uintptr_t)state & 15) == 0 &&
                     (PASS == 0 || ((uintptr_t)scratch & 15) == 0);
  auto load = [&](const float* from, float2 (&T)[M2_OWN][NPER / 2]) {
    if (whole) {
#pragma unroll
      for (int o = 0; o < M2_OWN; ++o)
#pragma unroll
        for (int i = 0; i < NPER / 4; ++i) {
          const float4 v = *reinterpret_cast<const float4*>(from + (size_t)o * N + part * NPER + 4 * i);
          T[o][2 * i] = make_float2(v.x, v.y);
          T[o][2 * i + 1] = make_float2(v.z, v.w);
        }
    } else {
#pragma unroll
      for (int o = 0; o < M2_OWN; ++o)
#pragma unroll
        for (int i = 0; i < NPER / 2; ++i) {
          const int row = part * NPER + 2 * i;
          const float* f = from + (size_t)o * N;
          T[o][i] = make_float2((col + o < P && row < N) ? f[row] : 0.f, (col + o < P && row + 1 < N) ? f[row + 1] : 0.f);
        }
    }
  };
  auto store = [&](float* to) {
    if (whole) {
#pragma unroll
      for (int o = 0; o < M2_OWN; ++o)
#pragma unroll
        for (int i = 0; i < NPER / 4; ++i)
          *reinterpret_cast<float4*>(to + (size_t)o * N + part * NPER + 4 * i) =
              make_float4(S[o][2 * i].x, S[o][2 * i].y, S[o][2 * i + 1].x, S[o][2 * i + 1].y);
      return;
    }
#pragma unroll
    for (int o = 0; o < M2_OWN; ++o)
#pragma unroll
      for (int i = 0; i < NPER / 2; ++i) {
        const int row = part * NPER + 2 * i;
        float* t = to + (size_t)o * N;
        if (col + o < P && row < N) t[row] = S[o][i].x;
        if (col + o < P && row + 1 < N) t[row + 1] = S[o][i].y;
      }
  };
  bool full = true;                        // reads C and writes y
  float* end = mine;                       // where the matrices go when the rows are done (nullptr: nowhere)
  float* product = nullptr;                // where the product of the decays goes
  if (PASS == 0) {
    load(mine, S);
  } else {
    const int length = (((n + segments - 1) / segments) + 15) & ~15;
    const int count = (n + length - 1) / length;
    if (seg >= count) return;
    const bool last = seg == count - 1;
    const size_t matrices = (size_t)heads * P * N;
    float* ends = scratch + (size_t)r * segments * matrices + ((size_t)head * P + col) * N;     // + seg * matrices
    float* products = scratch + (size_t)n_requests * segments * matrices + (size_t)r * segments * heads + head;
    first += seg * length;
    n = n - seg * length < length ? n - seg * length : length;
    if (PASS == 1) {
      if (seg == 0) {
        load(mine, S);
        end = last ? mine : ends;
      } else {
        if (last) return;
#pragma unroll
        for (int o = 0; o < M2_OWN; ++o)
#pragma unroll
          for (int i = 0; i < NPER / 2; ++i) S[o][i] = make_float2(0.f, 0.f);
        full = false;
        end = ends + (size_t)seg * matrices;
        if (blockIdx.x == 0 && threadIdx.x == 0) product = products + (size_t)seg * heads;
      }
    } else {
      if (seg == 0) return;
      load(ends, S);
      for (int j = 1; j < seg; ++j) {
        float2 local[M2_OWN][NPER / 2];
        load(ends + (size_t)j * matrices, local);
        const float decay = products[(size_t)j * heads];
        const float2 decay2 = make_float2(decay, decay);
#pragma unroll
        for (int o = 0; o < M2_OWN; ++o)
#pragma unroll
          for (int i = 0; i < NPER / 2; ++i) S[o][i] = __ffma2_rn(decay2, S[o][i], local[o][i]);
      }
      end = last ? mine : nullptr;
    }
  }
  __syncthreads();                         // the zeros are written before the first copies land
  // 16 bytes a copy where rows, lanes and channels come in whole 4s (a piece of 4 rows lies inside one part)
  const bool by16 = ((N | P | channels) & 3) == 0 && ((uintptr_t)xbc & 15) == 0;
  auto stage = [&](int run, int half) {    // the copies of a run's x, B and C, in flight when it returns
    const int here = n - run < RUN ? n - run : RUN;
    const int cols = P - col0 < M2_COLS ? P - col0 : M2_COLS;
    if (by16) {
      const int pieces = N >> 2;
      for (int i = threadIdx.x; i < here * pieces; i += M2_THREADS) {
        const int k = i / pieces, row = (i - k * pieces) << 2;
        const float* src = xbc + (size_t)(first + run + k) * channels + inner + group * N + row;
        const int at = (row / NPER) * PADDED + row % NPER;
        m2_copy16(&Bs[half][k][at], src);
        if (full) m2_copy16(&Cs[half][k][at], src + (size_t)groups * N);
      }
      const int across = cols >> 2;
      for (int i = threadIdx.x; i < here * across; i += M2_THREADS) {
        const int k = i / across, c = (i - k * across) << 2;
        m2_copy16(&xs[half][k][c], xbc + (size_t)(first + run + k) * channels + head * P + col0 + c);
      }
    } else {
      for (int i = threadIdx.x; i < here * N; i += M2_THREADS) {
        const int k = i / N, row = i - k * N;
        const float* src = xbc + (size_t)(first + run + k) * channels + inner + group * N + row;
        const int at = (row / NPER) * PADDED + row % NPER;
        m2_copy4(&Bs[half][k][at], src);
        if (full) m2_copy4(&Cs[half][k][at], src + (size_t)groups * N);
      }
      for (int i = threadIdx.x; i < here * cols; i += M2_THREADS) {
        const int k = i / cols, c = i - k * cols;
        m2_copy4(&xs[half][k][c], xbc + (size_t)(first + run + k) * channels + head * P + col0 + c);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  auto raw_step = [&](int run) {           // the raw step size of token run + threadIdx.x (asked for early)
    return threadIdx.x < RUN && run + (int)threadIdx.x < n
               ? to_float(proj[(size_t)(first + run + threadIdx.x) * ld + dt_at + head]) : 0.f;
  };
  auto keep_step = [&](float raw, int half) {
    if (threadIdx.x < RUN) {
      const float dt = m2_softplus(raw + bias);
      dts[half][threadIdx.x] = dt;
      decs[half][threadIdx.x] = expf(-a * dt);
    }
  };
  float decayed = 1.f;                     // the product of the decays of a run from zero
  stage(0, 0);
  keep_step(raw_step(0), 0);
  int half = 0;
  for (int run = 0; run < n; run += RUN, half ^= 1) {
    const int here = n - run < RUN ? n - run : RUN;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                       // this run has landed; the other half has been read to its end
    const bool more = run + RUN < n;
    float raw = 0.f;
    if (more) {
      stage(run + RUN, half ^ 1);
      raw = raw_step(run + RUN);
    }
    // one token of this thread's rows: S <- dec S + (dt x) B, and the rows' share of S^T C, for both columns
    // from one read of B and C.  Two rows an instruction (each lane an IEEE multiply or fused multiply-add of
    // its own), two sums of pairs a column so that the chain is half as long.
    auto token = [&](int k, float (&sum)[M2_OWN]) {
      const float dec = decs[half][k], dt = dts[half][k];
      const float4* b4 = reinterpret_cast<const float4*>(&Bs[half][k][part * PADDED]);
      const float4* c4 = reinterpret_cast<const float4*>(&Cs[half][k][part * PADDED]);
      const float2 dec2 = make_float2(dec, dec);
      float2 dtx2[M2_OWN], even[M2_OWN], odd[M2_OWN];
#pragma unroll
      for (int o = 0; o < M2_OWN; ++o) {
        const float dtx = dt * xs[half][k][mine_x + o];
        dtx2[o] = make_float2(dtx, dtx);
        even[o] = odd[o] = make_float2(0.f, 0.f);
      }
#pragma unroll
      for (int i = 0; i < NPER / 4; ++i) {
        const float4 b = b4[i], c = c4[i];
#pragma unroll
        for (int o = 0; o < M2_OWN; ++o) {
          S[o][2 * i] = __ffma2_rn(dec2, S[o][2 * i], __fmul2_rn(dtx2[o], make_float2(b.x, b.y)));
          S[o][2 * i + 1] = __ffma2_rn(dec2, S[o][2 * i + 1], __fmul2_rn(dtx2[o], make_float2(b.z, b.w)));
          even[o] = __ffma2_rn(S[o][2 * i], make_float2(c.x, c.y), even[o]);
          odd[o] = __ffma2_rn(S[o][2 * i + 1], make_float2(c.z, c.w), odd[o]);
        }
      }
#pragma unroll
      for (int o = 0; o < M2_OWN; ++o) {
        const float2 both = __fadd2_rn(even[o], odd[o]);
        sum[o] = both.x + both.y;
      }
    };
    int k = 0;
    if (PASS == 1 && !full) {              // from a zero start: the matrices and the product of the decays alone
      for (; k < here; ++k) {
        const float dec = decs[half][k], dt = dts[half][k];
        const float4* b4 = reinterpret_cast<const float4*>(&Bs[half][k][part * PADDED]);
        const float2 dec2 = make_float2(dec, dec);
        float2 dtx2[M2_OWN];
#pragma unroll
        for (int o = 0; o < M2_OWN; ++o) {
          const float dtx = dt * xs[half][k][mine_x + o];
          dtx2[o] = make_float2(dtx, dtx);
        }
#pragma unroll
        for (int i = 0; i < NPER / 4; ++i) {
          const float4 b = b4[i];
#pragma unroll
          for (int o = 0; o < M2_OWN; ++o) {
            S[o][2 * i] = __ffma2_rn(dec2, S[o][2 * i], __fmul2_rn(dtx2[o], make_float2(b.x, b.y)));
            S[o][2 * i + 1] = __ffma2_rn(dec2, S[o][2 * i + 1], __fmul2_rn(dtx2[o], make_float2(b.z, b.w)));
          }
        }
        decayed *= dec;
      }
    }
    // eight tokens at a time: the eight parts of a column add their shares of all eight in 4 + 2 + 1 exchanges
    // (a part passes on the half of the sums that the other side gathers), after which part j holds token j's
    // sum and writes it.  The pairs are those of the single token's rounds below, so a token's sum does not
    // depend on where in a run it falls.
    for (; k + M2_PARTS <= here; k += M2_PARTS) {
      float acc[M2_PARTS][M2_OWN];
#pragma unroll
      for (int j = 0; j < M2_PARTS; ++j) token(k + j, acc[j]);
#pragma unroll
      for (int width = M2_PARTS / 2; width >= 1; width >>= 1) {
        const bool upper = (part & width) != 0;
#pragma unroll
        for (int j = 0; j < width; ++j)
#pragma unroll
          for (int o = 0; o < M2_OWN; ++o) {
            const float send = upper ? acc[j][o] : acc[j + width][o], keep = upper ? acc[j + width][o] : acc[j][o];
            acc[j][o] = keep + __shfl_xor_sync(0xffffffffu, send, width);
          }
      }
#pragma unroll
      for (int o = 0; o < M2_OWN; ++o)
        if (col + o < P)
          y[(size_t)(first + run + k + part) * inner + head * P + col + o] = fmaf(d, xs[half][k + part][mine_x + o], acc[0][o]);
    }
    for (; k < here; ++k) {
      float acc[M2_OWN];
      token(k, acc);
#pragma unroll
      for (int o = 0; o < M2_OWN; ++o) {
        acc[o] += __shfl_xor_sync(0xffffffffu, acc[o], 4);
        acc[o] += __shfl_xor_sync(0xffffffffu, acc[o], 2);
        acc[o] += __shfl_xor_sync(0xffffffffu, acc[o], 1);
        if (part == 0 && col + o < P)
          y[(size_t)(first + run + k) * inner + head * P + col + o] = fmaf(d, xs[half][k][mine_x + o], acc[o]);
      }
    }
    if (more) keep_step(raw, half ^ 1);
  }
  if (end != nullptr) store(end);
  if (product != nullptr) *product = decayed;
}

// `segments` > 1: a request's rows run as that many segments side by side (two launches); `scratch` then has
// n_requests * segments * heads * (P * N + 1) floats.
TOKB200_API int tokb200_mamba2_scan(const float* xbc, int channels, const void* proj, int proj_dtype, int ld, int dt_at,
                                    const float* dt_bias, const float* a_log, const float* skip, int heads, int groups,
                                    int P, int N, float* state, long long stride, const int* q_start,
                                    const int* state_slot, int n_requests, float* y, float* scratch, int segments,
                                    cudaStream_t stream) {
  if (n_requests <= 0) return TOKB200_OK;
  if (heads <= 0 || groups <= 0 || heads % groups || P <= 0 || N <= 0 || N > 32 * M2_PARTS || heads > 65535 ||
      n_requests > 65535 || channels != heads * P + 2 * groups * N || (long long)heads * P * N > stride ||
      segments < 1 || (segments > 1 && scratch == nullptr) || (long long)n_requests * segments > 65535)
    return TOKB200_BAD_SIZE;
  const dim3 grid((P + M2_COLS - 1) / M2_COLS, heads, n_requests * segments);
#define LAUNCH_PASS(NPER, TI, PASS)                                                                               \
  launch_dependent(mamba2_scan_kernel<NPER, TI, PASS>, grid, dim3(M2_THREADS), 0, stream, xbc, channels,           \
                   (const TI*)proj, ld, dt_at, dt_bias, a_log, skip, heads, groups, P, N, state, stride, q_start,   \
                   state_slot, y, scratch, segments, n_requests)
#define LAUNCH(NPER, TI)                                              \
  {                                                                   \
    if (segments == 1) return LAUNCH_PASS(NPER, TI, 0);               \
    const int status = LAUNCH_PASS(NPER, TI, 1);                      \
    return status != TOKB200_OK ? status : LAUNCH_PASS(NPER, TI, 2);  \
  }
#define BY_SIZE(TI)                                   \
  if (N <= 4 * M2_PARTS) LAUNCH(4, TI);               \
  if (N <= 8 * M2_PARTS) LAUNCH(8, TI);               \
  if (N <= 16 * M2_PARTS) LAUNCH(16, TI);             \
  LAUNCH(32, TI)
  if (proj_dtype == TOKB200_F32) { BY_SIZE(float); }
  if (proj_dtype == TOKB200_BF16) { BY_SIZE(__nv_bfloat16); }
#undef BY_SIZE
#undef LAUNCH
#undef LAUNCH_PASS
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


// Four neighbouring lanes of the gate's pre-activation.
__device__ __forceinline__ float4 m2_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 m2_load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
  const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void m2_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void m2_store4(__nv_bfloat16* p, float4 v) {
  uint2 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
  h[0] = __floats2bfloat162_rn(v.x, v.y);
  h[1] = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = raw;
}
__device__ __forceinline__ float m2_silu(float z) { return z / (1.0f + expf(-z)); }

// The same for parts of whole 4s up to 2,048 lanes, everything aligned: four lanes a load, the part kept in
// registers between the sum and the scaling.
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
mamba2_out_norm4_kernel(const float* __restrict__ y, const TI* __restrict__ proj, int ld, int z_at,
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
  float4 kept[2];
  float squares = 0.f;
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int i = (threadIdx.x + k * blockDim.x) * 4;
    kept[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < width) {
      const float4 v = m2_load4(yr + i), z = m2_load4(zr + i);
      kept[k] = make_float4(v.x * m2_silu(z.x), v.y * m2_silu(z.y), v.z * m2_silu(z.z), v.w * m2_silu(z.w));
      squares = fmaf(kept[k].x, kept[k].x, squares);
      squares = fmaf(kept[k].y, kept[k].y, squares);
      squares = fmaf(kept[k].z, kept[k].z, squares);
      squares = fmaf(kept[k].w, kept[k].w, squares);
    }
  }
  const float inv = 1.0f / sqrtf(block_sum(squares, scratch) / (float)width + eps);
  TO* o = out + (size_t)t * inner + (size_t)g * width;
  const float* gr = gain + (size_t)g * width;
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int i = (threadIdx.x + k * blockDim.x) * 4;
    if (i < width) {
      const float4 w = m2_load4(gr + i);
      m2_store4(o + i, make_float4(kept[k].x * inv * w.x, kept[k].y * inv * w.y, kept[k].z * inv * w.z, kept[k].w * inv * w.w));
    }
  }
}

TOKB200_API int tokb200_mamba2_out_norm(const float* y, const void* proj, int proj_dtype, int ld, int z_at,
                                        const float* gain, float eps, int inner, int parts, const int* row_req,
                                        void* out, int out_dtype, int n_rows, cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (inner <= 0 || parts <= 0 || inner % parts || parts > 65535) return TOKB200_BAD_SIZE;
  const int width = inner / parts;
  const dim3 grid(n_rows, parts);
  const int z_size = proj_dtype == TOKB200_BF16 ? 2 : 4, o_size = out_dtype == TOKB200_BF16 ? 2 : 4;
  if (width % 4 == 0 && width <= 2048 && ld % 4 == 0 && z_at % 4 == 0 && (((uintptr_t)y | (uintptr_t)gain) & 15) == 0 &&
      ((uintptr_t)proj % (4 * z_size)) == 0 && ((uintptr_t)out % (4 * o_size)) == 0) {
    int threads4 = (width / 4 + 31) / 32 * 32;
    threads4 = threads4 > 256 ? 256 : threads4;
#define LAUNCH4(TI, TO)                                                                                              \
    return launch_dependent(mamba2_out_norm4_kernel<TI, TO>, grid, dim3(threads4), 0, stream, y, (const TI*)proj, ld, \
                            z_at, gain, eps, inner, parts, row_req, (TO*)out)
    if (proj_dtype == TOKB200_F32 && out_dtype == TOKB200_F32) LAUNCH4(float, float);
    if (proj_dtype == TOKB200_F32 && out_dtype == TOKB200_BF16) LAUNCH4(float, __nv_bfloat16);
    if (proj_dtype == TOKB200_BF16 && out_dtype == TOKB200_BF16) LAUNCH4(__nv_bfloat16, __nv_bfloat16);
    if (proj_dtype == TOKB200_BF16 && out_dtype == TOKB200_F32) LAUNCH4(__nv_bfloat16, float);
#undef LAUNCH4
  }
  int threads = (width + 31) / 32 * 32;
  threads = threads > 256 ? 256 : threads;
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
