// A feed-forward of routed experts, computed as ONE gated feed-forward whose inner lanes are the
// experts' lanes side by side (and a shared expert's behind them): every inner lane is scaled by its
// expert's share for the token, which is zero for an expert the token did not choose, so the down
// product over all lanes is the weighted sum of the chosen experts' outputs.
//
//   moe_route   the router's logits (32-bit sums; one more row for the shared expert's gate), then
//               share[t, e] = softmax over the `top` largest logits of token t (ties: the lower
//               index), zero elsewhere; share[t, experts] = sigmoid(the shared expert's gate logit)
//   moe_gate    act[t, c] = f(gate[t, c]) * up[t, c] * share[t, expert of lane c], f the activation
//
// moe_route knows a second way to score and choose (`score` = MOE_SCORE_SIGMOID): scores s =
// sigmoid(z); the CHOICE is made on s + correction (a learned number an expert, or none), and only
// among the experts of the `keep` best of `groups` equal groups of neighbouring experts, a group's
// worth being the sum of its two largest choice scores (the others count as minus infinity);
// share[t, e] = s[e] * scale for the chosen, not renormalized.  `shared` = 2: the shared expert's
// share is one (no gate row).  moe_gate knows a clamped activation (MOE_ACT_CLAMPED_SWISH): with
// g = min(gate, limit) and u = clamp(up, -limit, limit), g * sigmoid(alpha g) * (u + 1); the shared
// expert's lanes have a limit of their own.  With `on_input` the share multiplies the expert's INPUT instead
// of its output: the expert's first products are linear in their input, so its inner lanes are
// f(share * gate) * (share * up), and the down product adds the experts up unweighted.
#include "common.cuh"

enum : int { MOE_SCORE_SOFTMAX_OF_CHOSEN = 0, MOE_SCORE_SIGMOID = 1 };
enum : int { MOE_SHARED_NONE = 0, MOE_SHARED_GATED = 1, MOE_SHARED_ONE = 2 };
#define MOE_ACT_CLAMPED_SWISH TOKB200_ACT_COUNT

#define MOE_MAX_EXPERTS 1024

// h: the feed-forward's input [T, hidden] (float32, or its bfloat16 rounding); w: float32
// [experts + shared, hidden], the router's rows and behind them the shared expert's gate row.
// A block a token: its warps take the logits in turn (32-bit sums), thread 0 then chooses.
template <typename TI>
__global__ void __launch_bounds__(128)
moe_route_kernel(const TI* __restrict__ h, const float* __restrict__ w, int hidden, int experts, int top,
                 int shared_mode, float* __restrict__ share, int score, const float* __restrict__ correction,
                 int groups, int keep, float scale) {
  __shared__ float z[MOE_MAX_EXPERTS + 1];
  __shared__ float choice[MOE_MAX_EXPERTS];
  const int shared = shared_mode == MOE_SHARED_GATED ? 1 : 0;      // router rows behind the experts'
  const int columns = experts + (shared_mode != MOE_SHARED_NONE ? 1 : 0);
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TI* row = h + (size_t)t * hidden;
  for (int e = warp; e < experts + shared; e += blockDim.x >> 5) {
    const float* we = w + (size_t)e * hidden;
    float acc = 0.f;
    if (hidden % 128 == 0 && ((((uintptr_t)row) | ((uintptr_t)we)) & 15) == 0) {
      // four consecutive elements a lane and trip: one load of the input's, one of the router's row
      for (int i = lane * 4; i < hidden; i += 128) {
        const float4 wv = *reinterpret_cast<const float4*>(we + i);
        float4 hv;
        if (sizeof(TI) == 4) {
          hv = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(row) + i);
        } else {
          const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(row) + i);
          const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
          const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
          hv = make_float4(lo.x, lo.y, hi.x, hi.y);
        }
        acc = fmaf(hv.x, wv.x, acc);
        acc = fmaf(hv.y, wv.y, acc);
        acc = fmaf(hv.z, wv.z, acc);
        acc = fmaf(hv.w, wv.w, acc);
      }
    } else
    for (int i = lane; i < hidden; i += 32) acc = fmaf(to_float(row[i]), we[i], acc);
    acc = warp_sum(acc);
    if (lane == 0) z[e] = acc;
  }
  __syncthreads();
  float* out = share + (size_t)t * columns;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    out[e] = 0.f;
    if (score == MOE_SCORE_SIGMOID) {
      const float s = 1.0f / (1.0f + expf(-z[e]));
      z[e] = s;
      choice[e] = s + (correction ? correction[e] : 0.f);
    }
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  if (score == MOE_SCORE_SIGMOID) {
    // groups of neighbours: only the experts of the `keep` groups whose two largest choice scores
    // add up to the most can be chosen (ties: the lower group, the lower expert)
    const int size = experts / groups;
    unsigned open[MOE_MAX_EXPERTS / 32];
    for (int i = 0; i < (groups + 31) / 32; ++i) open[i] = 0u;
    if (keep < groups) {
      for (int k = 0; k < keep; ++k) {
        int best = -1;
        float worth = -INFINITY;
        for (int g = 0; g < groups; ++g) {
          if ((open[g >> 5] >> (g & 31)) & 1u) continue;
          float first = -INFINITY, second = -INFINITY;
          for (int e = g * size; e < (g + 1) * size; ++e) {
            const float c = choice[e];
            if (c > first) { second = first; first = c; } else if (c > second) { second = c; }
          }
          const float sum = size > 1 ? first + second : first;
          if (best < 0 || sum > worth) { best = g; worth = sum; }
        }
        if (best < 0) break;
        open[best >> 5] |= 1u << (best & 31);
      }
    }
    unsigned taken[MOE_MAX_EXPERTS / 32];
    for (int i = 0; i < (experts + 31) / 32; ++i) taken[i] = 0u;
    for (int k = 0; k < top; ++k) {
      int best = -1;
      float value = -INFINITY;
      for (int e = 0; e < experts; ++e) {
        const int g = e / size;
        if (keep < groups && !((open[g >> 5] >> (g & 31)) & 1u)) continue;
        if (!((taken[e >> 5] >> (e & 31)) & 1u) && (best < 0 || choice[e] > value)) {
          best = e;
          value = choice[e];
        }
      }
      if (best < 0) break;
      taken[best >> 5] |= 1u << (best & 31);
      out[best] = z[best] * scale;
    }
    if (shared_mode == MOE_SHARED_ONE) out[experts] = 1.0f;
    if (shared_mode == MOE_SHARED_GATED) out[experts] = 1.0f / (1.0f + expf(-z[experts]));
    return;
  }
  unsigned taken[MOE_MAX_EXPERTS / 32];
  for (int i = 0; i < (experts + 31) / 32; ++i) taken[i] = 0u;
  float highest = 0.f, sum = 0.f;
  for (int k = 0; k < top; ++k) {
    int best = -1;
    float value = -INFINITY;
    for (int e = 0; e < experts; ++e) {
      if (!((taken[e >> 5] >> (e & 31)) & 1u) && (best < 0 ? z[e] == z[e] : z[e] > value)) {
        best = e;
        value = z[e];
      }
    }
    if (best < 0) break;
    taken[best >> 5] |= 1u << (best & 31);
    if (k == 0) highest = value;
    const float weight = expf(value - highest);
    out[best] = weight;
    sum += weight;
  }
  for (int e = 0; e < experts; ++e)
    if ((taken[e >> 5] >> (e & 31)) & 1u) out[e] /= sum;
  if (shared_mode == MOE_SHARED_GATED) out[experts] = 1.0f / (1.0f + expf(-z[experts]));
  if (shared_mode == MOE_SHARED_ONE) out[experts] = 1.0f;
}

// act(gate) * up of one inner lane: the activations of every gated feed-forward, and the clamped one
__device__ __forceinline__ float moe_glu(int act, float g, float u, float limit, float alpha) {
  if (act == MOE_ACT_CLAMPED_SWISH) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
  }
  return gate_activation(act, g) * u;
}

// gu: [T, 2 I], gates in the first I columns, ups in the last; lanes 0 .. experts * ff belong to the
// routed experts (ff lanes each), the lanes behind to the shared expert.
template <typename T>
__global__ void moe_gate_kernel(const T* __restrict__ gu, const float* __restrict__ share, T* __restrict__ out,
                                int inner, int experts, int ff, int shared, int act, size_t n, float limit,
                                float shared_limit, float alpha, int on_input) {
  pdl_wait();
  pdl_launch();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const size_t t = i / inner;
    const int c = (int)(i % inner);
    const int e = c < experts * ff ? c / ff : experts;
    const float w = share[t * (experts + shared) + e];
    float value = 0.f;
    if (w != 0.f) {
      const float g = to_float(gu[t * 2 * inner + c]), u = to_float(gu[t * 2 * inner + inner + c]);
      const float lim = e < experts ? limit : shared_limit;
      value = on_input ? moe_glu(act, g * w, u * w, lim, alpha) : moe_glu(act, g, u, lim, alpha) * w;
    }
    out[i] = from_float<T>(value);
  }
}

// bfloat16, inner and expert widths in whole 8s: eight consecutive lanes (one expert's) a thread
__global__ void moe_gate_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, const float* __restrict__ share,
                                       __nv_bfloat16* __restrict__ out, int inner, int experts, int ff, int shared,
                                       int act, size_t n8, float limit, float shared_limit, float alpha,
                                       int on_input) {
  pdl_wait();
  pdl_launch();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const int per_row = inner / 8;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
    const size_t t = i / per_row;
    const int c = (int)(i % per_row) * 8;
    const int e = c < experts * ff ? c / ff : experts;
    const float w = share[t * (experts + shared) + e];
    uint4 packed = make_uint4(0u, 0u, 0u, 0u);
    if (w != 0.f) {
      const uint4 graw = *reinterpret_cast<const uint4*>(gu + t * 2 * inner + c);
      const uint4 uraw = *reinterpret_cast<const uint4*>(gu + t * 2 * inner + inner + c);
      const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&graw);
      const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uraw);
      __nv_bfloat162 h[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
        const float lim = e < experts ? limit : shared_limit;
        h[k] = on_input ? __floats2bfloat162_rn(moe_glu(act, g.x * w, u.x * w, lim, alpha),
                                                moe_glu(act, g.y * w, u.y * w, lim, alpha))
                        : __floats2bfloat162_rn(moe_glu(act, g.x, u.x, lim, alpha) * w,
                                                moe_glu(act, g.y, u.y, lim, alpha) * w);
      }
      packed = *reinterpret_cast<const uint4*>(h);
    }
    *reinterpret_cast<uint4*>(out + i * 8) = packed;
  }
}

TOKB200_API int tokb200_moe_route(const void* h, int h_dtype, const float* w, int hidden, int experts, int top,
                                  int shared, float* share, int n_rows, int score, const float* correction,
                                  int groups, int keep, float scale, cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (hidden <= 0 || experts <= 0 || experts > MOE_MAX_EXPERTS || top <= 0 || top > experts ||
      shared < MOE_SHARED_NONE || shared > MOE_SHARED_ONE ||
      (score != MOE_SCORE_SOFTMAX_OF_CHOSEN && score != MOE_SCORE_SIGMOID) || groups <= 0 || experts % groups ||
      keep <= 0 || keep > groups || (long long)keep * (experts / groups) < top)
    return TOKB200_BAD_SIZE;
  if (h_dtype == TOKB200_F32)
    return launch_dependent(moe_route_kernel<float>, dim3(n_rows), dim3(128), 0, stream, (const float*)h, w, hidden,
                            experts, top, shared, share, score, correction, groups, keep, scale);
  if (h_dtype == TOKB200_BF16)
    return launch_dependent(moe_route_kernel<__nv_bfloat16>, dim3(n_rows), dim3(128), 0, stream,
                            (const __nv_bfloat16*)h, w, hidden, experts, top, shared, share, score, correction, groups,
                            keep, scale);
  return TOKB200_BAD_DTYPE;
}

TOKB200_API int tokb200_moe_gate(const void* gu, const float* share, void* out, int dtype, int n_rows, int inner,
                                 int experts, int ff, int shared, int act, float limit, float shared_limit,
                                 float alpha, int on_input, cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (inner <= 0 || experts <= 0 || ff <= 0 || (long long)experts * ff > inner || act < 0 || act > MOE_ACT_CLAMPED_SWISH ||
      (!shared && (long long)experts * ff != inner))
    return TOKB200_BAD_SIZE;
  const size_t n = (size_t)n_rows * inner;
  const size_t blocks = (n + 255) / 256;
  const dim3 grid((unsigned)(blocks < 8192 ? blocks : 8192));
  if (dtype == TOKB200_F32)
    return launch_dependent(moe_gate_kernel<float>, grid, dim3(256), 0, stream, (const float*)gu, share, (float*)out,
                            inner, experts, ff, shared, act, n, limit, shared_limit, alpha, on_input);
  if (dtype == TOKB200_BF16 && inner % 8 == 0 && ff % 8 == 0 && (((uintptr_t)gu | (uintptr_t)out) & 15) == 0) {
    const size_t n8 = n / 8, blocks8 = (n8 + 255) / 256;
    return launch_dependent(moe_gate_bf16x8_kernel, dim3((unsigned)(blocks8 < 65535 ? blocks8 : 65535)), dim3(256), 0,
                            stream, (const __nv_bfloat16*)gu, share, (__nv_bfloat16*)out, inner, experts, ff, shared,
                            act, n8, limit, shared_limit, alpha, on_input);
  }
  if (dtype == TOKB200_BF16)
    return launch_dependent(moe_gate_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (const __nv_bfloat16*)gu,
                            share, (__nv_bfloat16*)out, inner, experts, ff, shared, act, n, limit, shared_limit, alpha,
                            on_input);
  return TOKB200_BAD_DTYPE;
}
