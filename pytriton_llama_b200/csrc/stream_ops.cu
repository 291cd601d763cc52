// Row-wise kernels on the float32 residual stream and around it: the scaled embedding with a
// sinusoidal position vector, the tanh cap of the logits, the clamped gated activation of a
// feed-forward, and the token-indexed side term of a layer.  All arithmetic is float32 (the
// position angles float64); T is the element type of projections' results and of weights.
#include "common.cuh"

namespace ptl {

// out[t, i] = table[ids[t], i] * scale (+ sin / cos of positions[t] * freq[i / 2] for even / odd i).
// An id outside [0, vocab) gives a zero row and raises *status.
template <typename T>
__global__ void embed_scaled_kernel(float* __restrict__ out, const T* __restrict__ table, const int* __restrict__ ids,
                                    const int* __restrict__ positions, const double* __restrict__ freq, int width, int vocab,
                                    float scale, int* __restrict__ status) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool bad = id < 0 || id >= vocab;
  if (bad && threadIdx.x == 0 && status) atomicExch(status, 1);
  const T* src = table + (size_t)(bad ? 0 : id) * width;
  const double pos = (double)positions[t];
  for (int pair = threadIdx.x; pair < (width + 1) / 2; pair += blockDim.x) {
    float a = 0.f, b = 0.f;
    if (freq) {
      double s, c;
      sincos(pos * freq[pair], &s, &c);
      a = (float)s;
      b = (float)c;
    }
    const int i = 2 * pair;
    out[(size_t)t * width + i] = (bad ? 0.f : to_f32(src[i]) * scale) + a;
    if (i + 1 < width) out[(size_t)t * width + i + 1] = (bad ? 0.f : to_f32(src[i + 1]) * scale) + b;
  }
}

__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap) {
  pdl_wait();
  pdl_launch_dependents();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

// gu [tokens, 2 * inter] (gate columns first) + bias: g = min(gate, limit), u = clamp(up, -limit, limit),
// out = g * sigmoid(alpha * g) * (u + up_shift).
template <typename T>
__global__ void clamped_glu_kernel(T* __restrict__ out, const T* __restrict__ gu, const float* __restrict__ bias, int inter,
                                   float limit, float alpha, float up_shift) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= inter) return;
  const T* row = gu + (size_t)t * 2 * inter;
  float g = to_f32(row[i]), u = to_f32(row[inter + i]);
  if (bias) { g += bias[i]; u += bias[inter + i]; }
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  out[(size_t)t * inter + i] = from_f32<T>(g / (1.0f + expf(-alpha * g)) * (u + up_shift));
}

__device__ __forceinline__ float gelu_tanh(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// A block takes TPB consecutive tokens.  s = residual + x + bias;  z = W_gate s;  g = gelu_tanh(z) * table[token, column + j];
// y = W_proj g;  residual = s + y * rsqrt(mean(y^2) + eps) * norm.   Every weight row is fetched once per block (16-byte
// packets where `vec_ok`) and used for all of the block's tokens.  Shared memory: TPB * (2 * width + dim) floats.
template <typename T, int TPB>
__global__ void __launch_bounds__(256)
token_side_kernel(float* __restrict__ residual, const T* __restrict__ x, const float* __restrict__ bias,
                  const int* __restrict__ tokens, const T* __restrict__ table, int table_ld, int column, int dim, int vocab,
                  const T* __restrict__ w_gate, const T* __restrict__ w_proj, const float* __restrict__ norm_w, int width,
                  float eps, int n_tokens, int vec_ok) {
  extern __shared__ __align__(16) float smem[];
  __shared__ float red[33];
  float* s = smem;
  float* y = s + (size_t)TPB * width;
  float* g = y + (size_t)TPB * width;
  constexpr int VN = Vec16<T>::N;
  pdl_wait();
  pdl_launch_dependents();
  const int t0 = blockIdx.x * TPB;
  const int nt = min(TPB, n_tokens - t0);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int k = 0; k < TPB; ++k) {
#pragma unroll 4
    for (int i = threadIdx.x; i < width; i += blockDim.x) {      // (four turns' loads are issued together)
      float v = 0.f;
      if (k < nt) {
        v = residual[(size_t)(t0 + k) * width + i];
        if (x) v += to_f32(x[(size_t)(t0 + k) * width + i]);
        if (bias) v += bias[i];
      }
      s[(size_t)k * width + i] = v;
    }
  }
  __syncthreads();
#pragma unroll (TPB == 1 ? 4 : 1)
  for (int j = warp; j < dim; j += nwarps) {       // (few tokens: four rows per turn, their packets fetched side by side)
    const T* wr = w_gate + (size_t)j * width;
    float acc[TPB];
#pragma unroll
    for (int k = 0; k < TPB; ++k) acc[k] = 0.f;
    if (vec_ok) {
#pragma unroll (TPB == 1 ? 4 : 1)
      for (int i = lane * VN; i < width; i += 32 * VN) {
        const Vec16<T> v = load16(wr + i);
#pragma unroll
        for (int k = 0; k < TPB; ++k) {
#pragma unroll
          for (int e = 0; e < VN; e += 4) {      // (16-byte reads of the row in shared memory: width is a multiple of VN here)
            const float4 a = *reinterpret_cast<const float4*>(s + (size_t)k * width + i + e);
            acc[k] = fmaf(a.x, v.get(e), acc[k]);
            acc[k] = fmaf(a.y, v.get(e + 1), acc[k]);
            acc[k] = fmaf(a.z, v.get(e + 2), acc[k]);
            acc[k] = fmaf(a.w, v.get(e + 3), acc[k]);
          }
        }
      }
    } else {
      for (int i = lane; i < width; i += 32) {
        const float wv = to_f32(wr[i]);
#pragma unroll
        for (int k = 0; k < TPB; ++k) acc[k] = fmaf(s[(size_t)k * width + i], wv, acc[k]);
      }
    }
#pragma unroll
    for (int k = 0; k < TPB; ++k) {
      const float z = warp_sum(acc[k]);
      if (lane == 0) {
        int tok = k < nt ? tokens[t0 + k] : 0;
        if (tok < 0 || tok >= vocab) tok = 0;
        g[k * dim + j] = gelu_tanh(z) * to_f32(table[(size_t)tok * table_ld + column + j]);
      }
    }
  }
  __syncthreads();
  float ss[TPB];
#pragma unroll
  for (int k = 0; k < TPB; ++k) ss[k] = 0.f;
#pragma unroll (TPB == 1 ? 4 : 1)
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const T* wr = w_proj + (size_t)i * dim;
    float acc[TPB];
#pragma unroll
    for (int k = 0; k < TPB; ++k) acc[k] = 0.f;
    if (vec_ok) {
      for (int j = 0; j < dim; j += VN) {
        const Vec16<T> v = load16(wr + j);
#pragma unroll
        for (int e = 0; e < VN; ++e) {
          const float wv = v.get(e);
#pragma unroll
          for (int k = 0; k < TPB; ++k) acc[k] = fmaf(g[k * dim + j + e], wv, acc[k]);
        }
      }
    } else {
      for (int j = 0; j < dim; ++j) {
        const float wv = to_f32(wr[j]);
#pragma unroll
        for (int k = 0; k < TPB; ++k) acc[k] = fmaf(g[k * dim + j], wv, acc[k]);
      }
    }
#pragma unroll
    for (int k = 0; k < TPB; ++k) {
      y[(size_t)k * width + i] = acc[k];
      ss[k] = fmaf(acc[k], acc[k], ss[k]);
    }
  }
#pragma unroll
  for (int k = 0; k < TPB; ++k) {
    const float total = block_sum(ss[k], red);
    if (k >= nt) continue;
    const float rrms = 1.0f / sqrtf(total / (float)width + eps);
#pragma unroll 4
    for (int i = threadIdx.x; i < width; i += blockDim.x)
      residual[(size_t)(t0 + k) * width + i] = s[(size_t)k * width + i] + y[(size_t)k * width + i] * rrms * norm_w[i];
  }
}

template <typename T>
int embed_scaled(float* out, const void* table, const int* ids, const int* positions, const double* freq, int tokens, int width,
                 int vocab, float scale, int* status, void* stream) {
  PTL_REQUIRE(tokens >= 0 && width > 0 && vocab > 0, "embed_scaled: bad sizes tokens=%d width=%d vocab=%d", tokens, width, vocab);
  if (tokens == 0) return 0;
  return launch_kernel("embed_scaled", embed_scaled_kernel<T>, dim3(tokens), dim3(128), 0, as_stream(stream), out, (const T*)table,
                       ids, positions, freq, width, vocab, scale, status);
}

template <typename T>
int clamped_glu(void* out, const void* gu, const float* bias, int tokens, int inter, float limit, float alpha, float up_shift,
                void* stream) {
  PTL_REQUIRE(tokens >= 0 && inter > 0 && limit > 0.f, "clamped_glu: bad sizes tokens=%d inter=%d limit=%f", tokens, inter, limit);
  PTL_REQUIRE(tokens <= 65535, "clamped_glu: at most 65535 rows per call, got %d", tokens);
  if (tokens == 0) return 0;
  return launch_kernel("clamped_glu", clamped_glu_kernel<T>, dim3((inter + 255) / 256, tokens), dim3(256), 0, as_stream(stream),
                       (T*)out, (const T*)gu, bias, inter, limit, alpha, up_shift);
}

template <typename T, int TPB>
int token_side_launch(float* residual, const void* x, const float* bias, const int* tokens, const void* table, int table_ld,
                      int column, int dim, int vocab, const void* w_gate, const void* w_proj, const float* norm_w, int n_tokens,
                      int width, float eps, int vec_ok, void* stream) {
  const size_t smem = (size_t)TPB * (2 * width + dim) * sizeof(float);
  static SmemRaised raised = {};
  if (smem > 48 * 1024)
    if (int rc = raise_shared_memory("token_side", token_side_kernel<T, TPB>, 200 * 1024, raised)) return rc;
  return launch_kernel("token_side", token_side_kernel<T, TPB>, dim3((n_tokens + TPB - 1) / TPB), dim3(256), smem,
                       as_stream(stream), residual, (const T*)x, bias, tokens, (const T*)table, table_ld, column, dim, vocab,
                       (const T*)w_gate, (const T*)w_proj, norm_w, width, eps, n_tokens, vec_ok);
}

template <typename T>
int token_side(float* residual, const void* x, const float* bias, const int* tokens, const void* table, int table_ld, int column,
               int dim, int vocab, const void* w_gate, const void* w_proj, const float* norm_w, int n_tokens, int width, float eps,
               void* stream) {
  PTL_REQUIRE(n_tokens >= 0 && width > 0 && dim > 0 && column >= 0 && column + dim <= table_ld && eps > 0.f,
              "token_side: bad sizes tokens=%d width=%d dim=%d column=%d of %d", n_tokens, width, dim, column, table_ld);
  if (n_tokens == 0) return 0;
  const size_t per_token = (size_t)(2 * width + dim) * sizeof(float);
  PTL_REQUIRE(per_token <= 200 * 1024, "token_side: width=%d, dim=%d do not fit the shared memory of a block", width, dim);
  constexpr int VN = Vec16<T>::N;
  const int vec_ok = width % VN == 0 && dim % VN == 0 && aligned16(w_gate) && aligned16(w_proj);
  // many tokens: four per block, so that a block's pass over the two weights serves four rows
  if (n_tokens >= 64 && 4 * per_token <= 200 * 1024)
    return token_side_launch<T, 4>(residual, x, bias, tokens, table, table_ld, column, dim, vocab, w_gate, w_proj, norm_w, n_tokens,
                                   width, eps, vec_ok, stream);
  return token_side_launch<T, 1>(residual, x, bias, tokens, table, table_ld, column, dim, vocab, w_gate, w_proj, norm_w, n_tokens,
                                 width, eps, vec_ok, stream);
}

}  // namespace ptl

PTL_EXPORT int ptl_softcap(float* x, long long n, float cap, void* stream) {
  PTL_REQUIRE(n >= 0 && cap > 0.f, "softcap: bad sizes n=%lld cap=%f", n, cap);
  if (n == 0) return 0;
  return ptl::launch_kernel("softcap", ptl::softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, ptl::as_stream(stream),
                            x, (size_t)n, cap);
}

#define PTL_STREAM_OPS(SUFFIX, TYPE)                                                                                              \
  PTL_EXPORT int ptl_embed_scaled##SUFFIX(float* out, const void* table, const int* ids, const int* positions, const double* freq, \
                                          int tokens, int width, int vocab, float scale, int* status, void* stream) {             \
    return ptl::embed_scaled<TYPE>(out, table, ids, positions, freq, tokens, width, vocab, scale, status, stream);                \
  }                                                                                                                               \
  PTL_EXPORT int ptl_clamped_glu##SUFFIX(void* out, const void* gu, const float* bias, int tokens, int inter, float limit,         \
                                         float alpha, float up_shift, void* stream) {                                             \
    return ptl::clamped_glu<TYPE>(out, gu, bias, tokens, inter, limit, alpha, up_shift, stream);                                  \
  }                                                                                                                               \
  PTL_EXPORT int ptl_token_side##SUFFIX(float* residual, const void* x, const float* bias, const int* tokens, const void* table,   \
                                        int table_ld, int column, int dim, int vocab, const void* w_gate, const void* w_proj,     \
                                        const float* norm_w, int n_tokens, int width, float eps, void* stream) {                  \
    return ptl::token_side<TYPE>(residual, x, bias, tokens, table, table_ld, column, dim, vocab, w_gate, w_proj, norm_w, n_tokens, \
                                 width, eps, stream);                                                                             \
  }
PTL_STREAM_OPS(_f32, float)
PTL_STREAM_OPS(_bf16, __nv_bfloat16)
