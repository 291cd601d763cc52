// Several copies of the residual stream: the write of one sub-layer and the read + RMS norm of the
// next in one pass over a token's row, and the tanh form of gelu.
//
// streams is float32 [tokens, S, width].  For output row m (token r = rows ? rows[m] : m), element w:
//   old_s  = streams[r, s, w]                     (or init[r, w] for every s when the copies start)
//   new_t  = sum_s mix[s, t] * old_s + out[t] * y[r, w]       (with y; else new = old)
//   streams[r, t, w] = new_t                      (unless rows are given: then nothing is stored)
//   u      = sum_t read[t] * new_t
//   normed[m, w] = u * rsqrt(mean_w(u^2) + eps) * weight[w]    rounded once to T
// Everything between the loads and the last rounding is float32.  A row is worked by one block, in
// the same order whatever else the step holds.
#include "common.cuh"

namespace ptl {

constexpr int kMostStreams = 16;   // the kernel is compiled for up to 4, 8 and 16 copies

// four neighbouring elements, from float32 (16 bytes) or bfloat16 (8 bytes)
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, float a, float b, float c, float d) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 t;
  t.x = *reinterpret_cast<const uint32_t*>(&lo);
  t.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = t;
}

template <typename T, typename Y, int kMaxStreams>
__global__ void __launch_bounds__(256)
stream_mix_norm_kernel(T* __restrict__ normed, float* __restrict__ streams, const T* __restrict__ init,
                       const Y* __restrict__ y, const float* __restrict__ mix, const float* __restrict__ out,
                       const float* __restrict__ read, const float* __restrict__ weight, const int* __restrict__ rows,
                       int S, int width, float eps, int vec_ok) {
  extern __shared__ float u_row[];           // [width]
  __shared__ float red[33];
  __shared__ float s_mix[kMaxStreams * kMaxStreams], s_out[kMaxStreams], s_read[kMaxStreams];
  // the small tables are weights: nothing of this step writes them
  if (threadIdx.x < S * S) s_mix[threadIdx.x] = mix ? mix[threadIdx.x] : ((threadIdx.x / S) == (threadIdx.x % S) ? 1.f : 0.f);
  if (threadIdx.x < S) {
    s_out[threadIdx.x] = out ? out[threadIdx.x] : 0.f;
    s_read[threadIdx.x] = read[threadIdx.x];
  }
  pdl_wait();
  pdl_launch_dependents();
  __syncthreads();
  const int m = blockIdx.x;
  const int r = rows ? rows[m] : m;
  float* st = streams + (size_t)r * S * width;
  const bool store = rows == nullptr;
  float ss = 0.f;
  if (vec_ok) {
    // four neighbouring elements per thread and turn: 16-byte packets of the copies, 8 or 16 bytes of T; the loads of a
    // turn are issued together and used afterwards
    for (int w = threadIdx.x * 4; w < width; w += blockDim.x * 4) {
      float old[kMaxStreams][4];
      if (init) {
        float v[4];
        load4(init + (size_t)r * width + w, v);
#pragma unroll
        for (int s = 0; s < kMaxStreams; ++s)
#pragma unroll
          for (int k = 0; k < 4; ++k) old[s][k] = v[k];
      } else {
#pragma unroll
        for (int s = 0; s < kMaxStreams; ++s) {
          if (s < S) {
            const float4 v = *reinterpret_cast<const float4*>(st + (size_t)s * width + w);
            old[s][0] = v.x; old[s][1] = v.y; old[s][2] = v.z; old[s][3] = v.w;
          } else {
            old[s][0] = old[s][1] = old[s][2] = old[s][3] = 0.f;
          }
        }
      }
      float yv[4] = {0.f, 0.f, 0.f, 0.f};
      if (y) load4(y + (size_t)r * width + w, yv);
      float u[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int t = 0; t < kMaxStreams; ++t) {
        if (t < S) {
          float nw[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            float acc;
            if (y) {
              acc = 0.f;
#pragma unroll
              for (int s = 0; s < kMaxStreams; ++s)
                if (s < S) acc = fmaf(s_mix[s * S + t], old[s][k], acc);
              acc = fmaf(s_out[t], yv[k], acc);
            } else {
              acc = old[t][k];
            }
            nw[k] = acc;
            u[k] = fmaf(s_read[t], acc, u[k]);
          }
          if (store && (y || init)) *reinterpret_cast<float4*>(st + (size_t)t * width + w) = make_float4(nw[0], nw[1], nw[2], nw[3]);
        }
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        u_row[w + k] = u[k];
        ss = fmaf(u[k], u[k], ss);
      }
    }
  } else
  for (int w = threadIdx.x; w < width; w += blockDim.x) {
    float old[kMaxStreams];
    if (init) {
      const float v = to_f32(init[(size_t)r * width + w]);
#pragma unroll
      for (int s = 0; s < kMaxStreams; ++s) old[s] = v;
    } else {
#pragma unroll
      for (int s = 0; s < kMaxStreams; ++s) old[s] = s < S ? st[(size_t)s * width + w] : 0.f;
    }
    float u = 0.f;
    if (y) {
      const float yv = to_f32(y[(size_t)r * width + w]);
#pragma unroll
      for (int t = 0; t < kMaxStreams; ++t) {
        if (t < S) {
          float acc = 0.f;
#pragma unroll
          for (int s = 0; s < kMaxStreams; ++s)
            if (s < S) acc = fmaf(s_mix[s * S + t], old[s], acc);
          acc = fmaf(s_out[t], yv, acc);
          if (store) st[(size_t)t * width + w] = acc;
          u = fmaf(s_read[t], acc, u);
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < kMaxStreams; ++t) {
        if (t < S) {
          if (init && store) st[(size_t)t * width + w] = old[t];
          u = fmaf(s_read[t], old[t], u);
        }
      }
    }
    u_row[w] = u;
    ss = fmaf(u, u, ss);
  }
  ss = block_sum(ss, red);
  const float rrms = 1.0f / sqrtf(ss / (float)width + eps);
  T* dst = normed + (size_t)m * width;
  if (vec_ok) {
    for (int w = threadIdx.x * 4; w < width; w += blockDim.x * 4) {
      const float4 wv = *reinterpret_cast<const float4*>(weight + w);
      store4(dst + w, u_row[w] * rrms * wv.x, u_row[w + 1] * rrms * wv.y, u_row[w + 2] * rrms * wv.z, u_row[w + 3] * rrms * wv.w);
    }
    return;
  }
  for (int w = threadIdx.x; w < width; w += blockDim.x) dst[w] = from_f32<T>(u_row[w] * rrms * weight[w]);
}

template <typename T, typename Y>
int stream_mix_norm(void* normed, float* streams, const void* init, const void* y, const float* mix, const float* out,
                    const float* read, const float* weight, const int* rows, int n_rows, int S, int width, float eps,
                    void* stream) {
  PTL_REQUIRE(n_rows >= 0 && width > 0 && eps > 0.f, "stream_mix_norm: bad sizes rows=%d width=%d", n_rows, width);
  PTL_REQUIRE(S >= 1 && S <= kMostStreams, "stream_mix_norm: %d copies of the stream, at most %d", S, kMostStreams);
  PTL_REQUIRE(streams && read && weight && normed, "stream_mix_norm: missing tensor");
  PTL_REQUIRE(!y || (mix && out), "stream_mix_norm: an output to write needs its mixing matrix and output vector");
  PTL_REQUIRE(!(init && y), "stream_mix_norm: the copies start from the embedding output or take a write, not both");
  if (n_rows == 0) return 0;
  const size_t smem = (size_t)width * sizeof(float);
  PTL_REQUIRE(smem <= 200 * 1024, "stream_mix_norm: width %d is too large", width);
  const int vec_ok = width % 4 == 0 && aligned16(streams) && aligned16(normed) && aligned16(weight) && (!init || aligned16(init)) &&
                     (!y || aligned16(y));
#define PTL_STREAM_LAUNCH(MS)                                                                                                  \
  {                                                                                                                            \
    static SmemRaised raised = {};                                                                                             \
    if (smem > 48 * 1024)                                                                                                      \
      if (int rc = raise_shared_memory("stream_mix_norm", stream_mix_norm_kernel<T, Y, MS>, 200 * 1024, raised)) return rc;   \
    return launch_kernel("stream_mix_norm", stream_mix_norm_kernel<T, Y, MS>, dim3(n_rows), dim3(256), smem, as_stream(stream), \
                         (T*)normed, streams, (const T*)init, (const Y*)y, mix, out, read, weight, rows, S, width, eps, vec_ok); \
  }
  if (S <= 4) PTL_STREAM_LAUNCH(4)
  if (S <= 8) PTL_STREAM_LAUNCH(8)
  PTL_STREAM_LAUNCH(16)
#undef PTL_STREAM_LAUNCH
}

// ------------------------------------------------------------------ gelu, tanh form
template <typename T>
__global__ void gelu_tanh_kernel(T* __restrict__ out, const T* __restrict__ x, long long n) {
  pdl_wait();
  pdl_launch_dependents();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float z = to_f32(x[i]);
  const float inner = 0.7978845608028654f * fmaf(0.044715f * z * z, z, z);
  out[i] = from_f32<T>(0.5f * z * (1.0f + tanhf(inner)));
}

template <typename T>
int gelu_tanh(void* out, const void* x, long long n, void* stream) {
  PTL_REQUIRE(n >= 0, "gelu_tanh: bad size");
  if (n == 0) return 0;
  return launch_kernel("gelu_tanh", gelu_tanh_kernel<T>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, as_stream(stream),
                       (T*)out, (const T*)x, n);
}

}  // namespace ptl

#define PTL_STREAMS(SUFFIX, TYPE)                                                                                                   \
  PTL_EXPORT int ptl_stream_mix_norm##SUFFIX(void* normed, float* streams, const void* init, const void* y, int y_is_f32,            \
                                             const float* mix, const float* out, const float* read, const float* weight,            \
                                             const int* rows, int n_rows, int S, int width, float eps, void* stream) {              \
    if (y_is_f32)                                                                                                                   \
      return ptl::stream_mix_norm<TYPE, float>(normed, streams, init, y, mix, out, read, weight, rows, n_rows, S, width, eps, stream); \
    return ptl::stream_mix_norm<TYPE, TYPE>(normed, streams, init, y, mix, out, read, weight, rows, n_rows, S, width, eps, stream); \
  }                                                                                                                                 \
  PTL_EXPORT int ptl_gelu_tanh##SUFFIX(void* out, const void* x, long long n, void* stream) {                                        \
    return ptl::gelu_tanh<TYPE>(out, x, n, stream);                                                                                 \
  }
PTL_STREAMS(_f32, float)
PTL_STREAMS(_bf16, __nv_bfloat16)
