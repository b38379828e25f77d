// Queries, keys and values of an attention layer whose key and value heads differ in size, from one
// stacked product: the projection's bias, the rotation of the leading `rot_dims` lanes of every query
// and key head in the interleaved form (lane 2i pairs with lane 2i + 1; the pair (u, v) at position p
// becomes (u cos a - v sin a, v cos a + u sin a), a = float32(p) * inv_freq[i], or, where the frequencies come
// in 64-bit (`inv_freq64`), the 64-bit product brought into one turn before it is rounded), and the write of the
// token's keys and values into its cache slot.  Cache rows and query rows have `row` lanes a head,
// row >= max(dim, vdim): keys and queries fill the first `dim` lanes, values the first `vdim`, the
// rest is written as zero, so that kernels which take one head size serve both.
//
// proj: [T, ld]; columns at .. : q (heads * dim), k (kv_heads * dim), v (kv_heads * vdim).
// bias: float32, indexed like proj's columns from `at` on (or null).  A block a token.
//
// With `q_gain` / `k_gain` (float32, one a column of q and of k): before the rotation the token's
// whole q projection (all heads at once) is divided by its root mean square, eps inside the root,
// and multiplied by q_gain; the same for k.  With `temp` (float32, one a query head): the head's
// queries are multiplied by it, which multiplies the head's scores.  All of it in 32-bit.
//
// `half_layout`: the rotated lanes pair in the half form instead (lane i with lane i + rot_dims / 2, both
// turned by the angle of frequency i).  `head_norm`: after the rotation every query head and every key
// head is divided by its own root mean square over its `dim` lanes (`head_eps` inside the root, no gain).
// A rotation turns pairs and leaves each pair's sum of squares as it was, so a head's mean square is
// taken of its lanes before the rotation, a warp a head, and kept in shared memory.  A token's sines and
// cosines are computed once a frequency into shared memory (every head turns by the same angles).  `kv_heads` = 0: the
// projection holds queries only (a layer that reads another layer's cache): nothing is written but q_out.
//
// attention_gate: out[t, h, l] *= sigmoid(proj[t, at + h * vdim + l]), l < vdim, on rows of `row` lanes a
// head: a gate on the heads' outputs that is one more projection of the mixer's input.
#include "common.cuh"

__device__ __forceinline__ void rs_store4(float* dst, const float v[4]) {
  *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void rs_store4(__nv_bfloat16* dst, const float v[4]) {
  __nv_bfloat162 h[2] = {__floats2bfloat162_rn(v[0], v[1]), __floats2bfloat162_rn(v[2], v[3])};
  *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(h);
}
// four consecutive columns of a float32 product from `col` on: + bias, then * inv * gain (each where given)
__device__ __forceinline__ void rs_load4(const float* in, int col, const float* bias, const float* gain, int gain_col,
                                         float inv, float v[4]) {
  const float4 x = *reinterpret_cast<const float4*>(in + col);
  v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  if (bias != nullptr) {
    const float4 b = *reinterpret_cast<const float4*>(bias + col);
    v[0] += b.x; v[1] += b.y; v[2] += b.z; v[3] += b.w;
  }
  if (gain != nullptr) {
    const float4 g = *reinterpret_cast<const float4*>(gain + gain_col);
    v[0] = v[0] * inv * g.x; v[1] = v[1] * inv * g.y; v[2] = v[2] * inv * g.z; v[3] = v[3] * inv * g.w;
  }
}

template <typename TI, typename T>
__global__ void qkv_rotate_store_kernel(const TI* __restrict__ proj, int ld, int at, const float* __restrict__ bias,
                                        const float* __restrict__ inv_freq,
                                        const double* __restrict__ inv_freq64, int rot_dims,
                                        const int* __restrict__ pos, const int* __restrict__ slot,
                                        const int* __restrict__ row_req, T* __restrict__ q_out,
                                        T* __restrict__ k_pool, T* __restrict__ v_pool, int heads, int kv_heads,
                                        int dim, int vdim, int row, const float* __restrict__ q_gain,
                                        const float* __restrict__ k_gain, float eps, const float* __restrict__ temp,
                                        int half_layout, int head_norm, float head_eps, int quads) {
  // shared memory: a token's cosines and sines, one pair a frequency (every head turns by the same
  // angles), then the heads' inverse root mean squares (with `head_norm`)
  extern __shared__ float shared[];
  __shared__ float scratch[33];
  const int half = rot_dims >> 1;
  float* cosine = shared;
  float* sine = shared + half;
  float* head_inv = shared + 2 * half;
  const int t = blockIdx.x;
  const int r = row_req[t];
  const int p = pos[t];
  const int where = slot ? slot[t] : -1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float angle;
    if (inv_freq64 != nullptr) {       // the product and its reduction to one turn in 64-bit: good to 1e-7 at any position
      double a = (double)p * inv_freq64[i];
      a -= 6.283185307179586476925 * rint(a * 0.15915494309189533577);
      angle = (float)a;
    } else {
      angle = (float)p * inv_freq[i];
    }
    sincosf(angle, &sine[i], &cosine[i]);
  }
  pdl_wait();
  pdl_launch();
  if (r < 0) return;
  const TI* in = proj + (size_t)t * ld + at;
  float q_inv = 1.f, k_inv = 1.f;
  if (q_gain != nullptr || k_gain != nullptr) {         // root mean squares over the whole projections
    float qs = 0.f, ks = 0.f;
    if (sizeof(TI) == 4 && quads) {
      for (int col = threadIdx.x * 4; col < (heads + kv_heads) * dim; col += blockDim.x * 4) {
        float v[4];
        rs_load4(reinterpret_cast<const float*>(in), col, bias, nullptr, 0, 1.f, v);
        const float sum = fmaf(v[3], v[3], fmaf(v[2], v[2], fmaf(v[1], v[1], v[0] * v[0])));
        if (col < heads * dim) qs += sum; else ks += sum;
      }
    } else
    for (int col = threadIdx.x; col < (heads + kv_heads) * dim; col += blockDim.x) {
      const float v = to_float(in[col]) + (bias ? bias[col] : 0.f);
      if (col < heads * dim) qs = fmaf(v, v, qs); else ks = fmaf(v, v, ks);
    }
    qs = block_sum(qs, scratch);
    ks = block_sum(ks, scratch);
    if (q_gain != nullptr) q_inv = 1.0f / sqrtf(qs / (float)(heads * dim) + eps);
    if (k_gain != nullptr) k_inv = 1.0f / sqrtf(ks / (float)(kv_heads * dim) + eps);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  if (head_norm) {                                      // a warp a head: the mean square of its lanes
    for (int head = warp; head < heads + kv_heads; head += warps) {
      const bool query = head < heads;
      const float* gain = query ? q_gain : k_gain;
      const float inv = query ? q_inv : k_inv;
      const int first = query ? 0 : heads * dim;
      float sum = 0.f;
      if (sizeof(TI) == 4 && quads) {
        for (int l = lane * 4; l < dim; l += 128) {
          float v[4];
          rs_load4(reinterpret_cast<const float*>(in), head * dim + l, bias, gain, head * dim + l - first, inv, v);
          sum += fmaf(v[3], v[3], fmaf(v[2], v[2], fmaf(v[1], v[1], v[0] * v[0])));
        }
      } else
      for (int l = lane; l < dim; l += 32) {
        const int col = head * dim + l;
        float v = to_float(in[col]) + (bias ? bias[col] : 0.f);
        if (gain != nullptr) v = v * inv * gain[col - first];
        sum = fmaf(v, v, sum);
      }
      sum = warp_sum(sum);
      if (lane == 0) head_inv[head] = 1.0f / sqrtf(sum / (float)dim + head_eps);
    }
  }
  __syncthreads();                                      // the angles' table (and the heads' norms) are written
  // a warp a head.  Where every size is whole 4s and everything lies on 16 bytes (`quads`, float32 products):
  // four consecutive lanes a thread, 16-byte loads, the same arithmetic lane by lane as below.
  if (sizeof(TI) == 4 && quads) {
    const float* fin = reinterpret_cast<const float*>(in);
    for (int head = warp; head < heads + 2 * kv_heads; head += warps) {
      if (head < heads + kv_heads) {
        const bool query = head < heads;
        T* dst = query ? q_out + ((size_t)t * heads + head) * row
                       : (where >= 0 ? k_pool + ((size_t)where * kv_heads + (head - heads)) * row : nullptr);
        if (dst == nullptr) continue;
        const float* gain = query ? q_gain : k_gain;
        const float inv = query ? q_inv : k_inv;
        const int first = query ? 0 : heads * dim;
        const float after = (head_norm ? head_inv[head] : 1.f);
        const float heat = (query && temp != nullptr) ? temp[head] : 1.f;
        for (int l = lane * 4; l < row; l += 128) {
          float v[4] = {0.f, 0.f, 0.f, 0.f};
          if (l < dim) {
            const int col = head * dim + l;
            rs_load4(fin, col, bias, gain, col - first, inv, v);
            if (l < rot_dims) {
              if (half_layout) {
                const bool second = l >= half;
                const int mate = second ? col - half : col + half;
                const int f = second ? l - half : l;
                float m[4];
                rs_load4(fin, mate, bias, gain, mate - first, inv, m);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  v[j] = second ? v[j] * cosine[f + j] + m[j] * sine[f + j] : v[j] * cosine[f + j] - m[j] * sine[f + j];
              } else {
                const int f = l >> 1;
                const float a0 = v[0], a1 = v[1], a2 = v[2], a3 = v[3];
                v[0] = a0 * cosine[f] - a1 * sine[f];
                v[1] = a1 * cosine[f] + a0 * sine[f];
                v[2] = a2 * cosine[f + 1] - a3 * sine[f + 1];
                v[3] = a3 * cosine[f + 1] + a2 * sine[f + 1];
              }
            }
            if (head_norm) {
#pragma unroll
              for (int j = 0; j < 4; ++j) v[j] *= after;
            }
            if (query && temp != nullptr) {
#pragma unroll
              for (int j = 0; j < 4; ++j) v[j] *= heat;
            }
          }
          rs_store4(dst + l, v);
        }
      } else if (where >= 0) {
        const int g = head - heads - kv_heads;
        T* dst = v_pool + ((size_t)where * kv_heads + g) * row;
        const int col0 = (heads + kv_heads) * dim + g * vdim;
        for (int l = lane * 4; l < row; l += 128) {
          float v[4] = {0.f, 0.f, 0.f, 0.f};
          if (l < vdim) rs_load4(fin, col0 + l, bias, nullptr, 0, 1.f, v);
          rs_store4(dst + l, v);
        }
      }
    }
    return;
  }
  // a lane every 32nd lane of its row
  for (int head = warp; head < heads + 2 * kv_heads; head += warps) {
    if (head < heads + kv_heads) {                       // a query or key head: bias, norms, rotation
      const bool query = head < heads;
      T* dst = query ? q_out + ((size_t)t * heads + head) * row
                     : (where >= 0 ? k_pool + ((size_t)where * kv_heads + (head - heads)) * row : nullptr);
      if (dst == nullptr) continue;
      const float* gain = query ? q_gain : k_gain;
      const float inv = query ? q_inv : k_inv;
      const int first = query ? 0 : heads * dim;         // the gains are indexed inside q and inside k
      const float after = (head_norm ? head_inv[head] : 1.f);
      const float heat = (query && temp != nullptr) ? temp[head] : 1.f;
      for (int l = lane; l < row; l += 32) {
        float value = 0.f;
        if (l < dim) {
          const int col = head * dim + l;
          value = to_float(in[col]) + (bias ? bias[col] : 0.f);
          if (gain != nullptr) value = value * inv * gain[col - first];
          if (l < rot_dims) {
            const bool second = half_layout ? l >= half : (l & 1);      // the pair's second lane
            const int mate = half_layout ? (second ? col - half : col + half) : (col ^ 1);
            float other = to_float(in[mate]) + (bias ? bias[mate] : 0.f);
            if (gain != nullptr) other = other * inv * gain[mate - first];
            const int f = half_layout ? (second ? l - half : l) : (l >> 1);
            const float c = cosine[f], sn = sine[f];
            value = second ? value * c + other * sn : value * c - other * sn;
          }
          if (head_norm) value *= after;
          if (query && temp != nullptr) value *= heat;
        }
        dst[l] = from_float<T>(value);
      }
    } else if (where >= 0) {
      const int g = head - heads - kv_heads;
      T* dst = v_pool + ((size_t)where * kv_heads + g) * row;
      const int col0 = (heads + kv_heads) * dim + g * vdim;
      for (int l = lane; l < row; l += 32) {
        float value = 0.f;
        if (l < vdim) value = to_float(in[col0 + l]) + (bias ? bias[col0 + l] : 0.f);
        dst[l] = from_float<T>(value);
      }
    }
  }
}

TOKB200_API int tokb200_qkv_rotate_store(const void* proj, int proj_dtype, int ld, int at, const float* bias,
                                         const float* inv_freq, const double* inv_freq64, int rot_dims,
                                         const int* pos, const int* slot,
                                         const int* row_req, void* q_out, void* k_pool, void* v_pool,
                                         int out_dtype, int n_rows, int heads, int kv_heads, int dim, int vdim,
                                         int row, const float* q_gain, const float* k_gain, float eps,
                                         const float* temp, int half_layout, int head_norm, float head_eps,
                                         cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (kv_heads == 0 && (slot != nullptr || k_gain != nullptr)) return TOKB200_BAD_SIZE;
  const size_t smem = (size_t)(rot_dims + (head_norm ? heads + kv_heads : 0)) * sizeof(float);
  if (smem > 40000) return TOKB200_BAD_SIZE;
  // four lanes a thread: float32 products whose columns, heads and rows are whole 4s (rotated lanes whole 8s, so
  // that a quad lies inside one half) with every pointer on 16 bytes
  const uintptr_t all = (uintptr_t)proj | (uintptr_t)bias | (uintptr_t)q_gain | (uintptr_t)k_gain | (uintptr_t)q_out |
                        (uintptr_t)k_pool | (uintptr_t)v_pool;
  const int quads = proj_dtype == TOKB200_F32 && dim % 4 == 0 && vdim % 4 == 0 && row % 4 == 0 && rot_dims % 8 == 0 &&
                    at % 4 == 0 && ld % 4 == 0 && (all & 15) == 0;
  if (heads <= 0 || kv_heads < 0 || dim <= 0 || vdim <= 0 || row < dim || row < vdim || rot_dims < 0 ||
      rot_dims % 2 || rot_dims > dim || (rot_dims > 0 && inv_freq == nullptr && inv_freq64 == nullptr))
    return TOKB200_BAD_SIZE;
#define LAUNCH(TI, T)                                                                                         \
  return launch_dependent(qkv_rotate_store_kernel<TI, T>, dim3(n_rows), dim3(256), smem, stream,              \
                          (const TI*)proj, ld, at, bias, inv_freq, inv_freq64, rot_dims, pos, slot, row_req,  \
                          (T*)q_out,                                                                          \
                          (T*)k_pool, (T*)v_pool, heads, kv_heads, dim, vdim, row, q_gain, k_gain, eps, temp, \
                          half_layout, head_norm, head_eps, quads)
  if (proj_dtype == TOKB200_F32 && out_dtype == TOKB200_F32) LAUNCH(float, float);
  if (proj_dtype == TOKB200_F32 && out_dtype == TOKB200_BF16) LAUNCH(float, __nv_bfloat16);
  if (proj_dtype == TOKB200_BF16 && out_dtype == TOKB200_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  if (proj_dtype == TOKB200_BF16 && out_dtype == TOKB200_F32) LAUNCH(__nv_bfloat16, float);
#undef LAUNCH
  return TOKB200_BAD_DTYPE;
}

// out: [T, heads * row] in place; proj: [T, ld], the gate's columns at .. (heads * vdim)
template <typename TI, typename T>
__global__ void attention_gate_kernel(T* __restrict__ out, const TI* __restrict__ proj, int ld, int at, int heads,
                                      int vdim, int row, size_t n) {
  pdl_wait();
  pdl_launch();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const int per_row = heads * vdim;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const size_t t = i / per_row;
    const int c = (int)(i % per_row), head = c / vdim, l = c % vdim;
    const float g = to_float(proj[t * ld + at + c]);
    T* o = out + (t * heads + head) * row + l;
    *o = from_float<T>(to_float(*o) / (1.0f + expf(-g)));
  }
}

// float32 pre-activations, bfloat16 outputs, value heads in whole 8s: eight consecutive lanes a thread
__global__ void attention_gate_f32_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ proj, int ld,
                                                 int at, int heads, int vdim, int row, size_t n8) {
  pdl_wait();
  pdl_launch();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const int per_head = vdim / 8, per_row = heads * per_head;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
    const size_t t = i / per_row;
    const int c = (int)(i % per_row), head = c / per_head, l = (c % per_head) * 8;
    const float* g = proj + t * ld + at + head * vdim + l;
    const float4 g0 = *reinterpret_cast<const float4*>(g), g1 = *reinterpret_cast<const float4*>(g + 4);
    __nv_bfloat16* o = out + (t * heads + head) * row + l;
    uint4 raw = *reinterpret_cast<const uint4*>(o);
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
    const float gate[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 v = __bfloat1622float2(h[k]);
      h[k] = __floats2bfloat162_rn(v.x / (1.0f + expf(-gate[2 * k])), v.y / (1.0f + expf(-gate[2 * k + 1])));
    }
    *reinterpret_cast<uint4*>(o) = raw;
  }
}

TOKB200_API int tokb200_attention_gate(void* out, int out_dtype, const void* proj, int proj_dtype, int ld, int at,
                                       int n_rows, int heads, int vdim, int row, cudaStream_t stream) {
  if (n_rows <= 0) return TOKB200_OK;
  if (heads <= 0 || vdim <= 0 || row < vdim || at < 0 || ld < at + heads * vdim) return TOKB200_BAD_SIZE;
  const size_t n = (size_t)n_rows * heads * vdim;
  if (proj_dtype == TOKB200_F32 && out_dtype == TOKB200_BF16 && vdim % 8 == 0 && row % 8 == 0 && ld % 4 == 0 &&
      at % 4 == 0 && ((uintptr_t)out & 15) == 0 && ((uintptr_t)proj & 15) == 0) {
    const size_t n8 = n / 8, blocks8 = (n8 + 255) / 256;
    return launch_dependent(attention_gate_f32_bf16x8_kernel, dim3((unsigned)(blocks8 < 65535 ? blocks8 : 65535)),
                            dim3(256), 0, stream, (__nv_bfloat16*)out, (const float*)proj, ld, at, heads, vdim, row, n8);
  }
  const size_t blocks = (n + 255) / 256;
  const dim3 grid((unsigned)(blocks < 8192 ? blocks : 8192));
#define LAUNCH(TI, T)                                                                                          \
  return launch_dependent(attention_gate_kernel<TI, T>, grid, dim3(256), 0, stream, (T*)out, (const TI*)proj, ld, at, \
                          heads, vdim, row, n)
  if (proj_dtype == TOKB200_F32 && out_dtype == TOKB200_F32) LAUNCH(float, float);
  if (proj_dtype == TOKB200_F32 && out_dtype == TOKB200_BF16) LAUNCH(float, __nv_bfloat16);
  if (proj_dtype == TOKB200_BF16 && out_dtype == TOKB200_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  if (proj_dtype == TOKB200_BF16 && out_dtype == TOKB200_F32) LAUNCH(__nv_bfloat16, float);
#undef LAUNCH
  return TOKB200_BAD_DTYPE;
}
