// Attention inside blocks of positions over the paged cache, with a distance bias on the scores, weights
// mixed between heads after the softmax, and values that are normed before they are stored.
//
// A page of the cache holds its keys, then its values: element (g, offset, e) of the keys lies at
// page * page_stride + (g * page_size + offset) * d + e, of the values at
// page * page_stride + G * page_size * d + (g * page_size + offset) * dv + e, page_stride = G * page_size * (d + dv).
// Scores, weights and all sums are float32; T is the element type of q, of the cache and of the result.
#include "common.cuh"

namespace ptl {

// k (+ bias) and v (+ bias, then divided by its root mean square per head when eps > 0) of every token go to
// the token's slot (page * page_size + offset; -1: not stored).  qkv rows: [q: H * d | k: G * d | v: G * dv].
template <typename T>
__global__ void __launch_bounds__(128)
kv_write_normed_kernel(T* __restrict__ cache, const T* __restrict__ qkv, const float* __restrict__ bias,
                       const int* __restrict__ slots, int H, int G, int d, int dv, int page_size, long long num_slots, float eps) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const long long slot = slots[t];
  if (slot < 0 || slot >= num_slots) return;
  const size_t page = (size_t)(slot / page_size), off = (size_t)(slot % page_size);
  const int ld = H * d + G * (d + dv);
  const T* row = qkv + (size_t)t * ld;
  T* kp = cache + page * (size_t)G * page_size * (d + dv);
  T* vp = kp + (size_t)G * page_size * d;
#pragma unroll 4
  for (int i = threadIdx.x; i < G * d; i += blockDim.x) {
    const int g = i / d, e = i % d;
    const float v = to_f32(row[H * d + i]) + (bias ? bias[H * d + i] : 0.f);
    kp[((size_t)g * page_size + off) * d + e] = from_f32<T>(v);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int g = warp; g < G; g += nwarps) {
    const int base = (H + G) * d + g * dv;
    float ss = 0.f;
#pragma unroll 4
    for (int e = lane; e < dv; e += 32) {
      const float v = to_f32(row[base + e]) + (bias ? bias[base + e] : 0.f);
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float f = eps > 0.f ? 1.0f / sqrtf(ss / (float)dv + eps) : 1.0f;
#pragma unroll 4
    for (int e = lane; e < dv; e += 32) {
      const float v = to_f32(row[base + e]) + (bias ? bias[base + e] : 0.f);
      vp[((size_t)g * page_size + off) * dv + e] = from_f32<T>(v * f);
    }
  }
}

constexpr int kMaxMixedHeads = 128;     // heads whose weights can be mixed (a thread holds one key's column of them)

// One block per query token.  Keys j = lo .. p of the token's request, lo = p - p % chunk (0 without chunks):
//   score_h(j) = (q_h + bias) . k_j * scale - r1[h] * log1p(r2[h] * (p - j));   w_h = softmax_j;
//   w'_h = sum_g talk[h, g] w_g;   out_h = out_scale * sum_j w'_h(j) v_j.
// Shared memory: max_keys page addresses, the query (H * d floats), H * max_keys weights.
template <typename T>
__global__ void __launch_bounds__(256)
chunk_attention_kernel(T* __restrict__ out, int out_ld, int column, const T* __restrict__ qkv, int q_ld,
                       const float* __restrict__ q_bias, const T* __restrict__ cache, const int* __restrict__ block_table,
                       int table_width, const int* __restrict__ tok_req, const int* __restrict__ positions, int H, int G, int d,
                       int dv, int page_size, float scale, int chunk, const float* __restrict__ r1, const float* __restrict__ r2,
                       const float* __restrict__ talk, int max_keys, int num_pages, float out_scale, int vec_ok) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  long long* page_at = reinterpret_cast<long long*>(smem_raw);       // first element of the page that holds key j, -1: none
  float* q = reinterpret_cast<float*>(page_at + max_keys);
  float* w = q + H * d;
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int r = tok_req[t];
  if (r < 0) return;
  const int p = positions[t];
  const int lo = chunk > 0 ? p - p % chunk : 0;
  const int n = min(p - lo + 1, max_keys);
  const int group = H / G;
  const size_t page_stride = (size_t)G * page_size * (d + dv);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll 4
  for (int i = threadIdx.x; i < H * d; i += blockDim.x)      // (four turns' loads are issued together)
    q[i] = to_f32(qkv[(size_t)t * q_ld + i]) + (q_bias ? q_bias[i] : 0.f);
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    const int pos = lo + j;
    const int page = block_table[(size_t)r * table_width + pos / page_size];
    page_at[j] = (page >= 0 && page < num_pages) ? (long long)((size_t)page * page_stride) : -1;
  }
  __syncthreads();
  // scores: one (kv head, key) pair per thread and turn, for up to four of the kv head's query heads at a time, so that
  // a key row is fetched once for them; consecutive threads take consecutive keys
  for (int i = threadIdx.x; i < G * n; i += blockDim.x) {
    const int c = i / n, j = i % n;
    const bool there = page_at[j] >= 0;
    const T* kr = cache + (there ? page_at[j] : 0) + ((size_t)c * page_size + (lo + j) % page_size) * d;
    for (int h0 = c * group; h0 < (c + 1) * group; h0 += 4) {
      const int nh = min(4, (c + 1) * group - h0);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      if (there && vec_ok) {                            // 16-byte packets of the key row and of the queries
        constexpr int VN = Vec16<T>::N;
#pragma unroll 8
        for (int e = 0; e < d; e += VN) {
          const Vec16<T> kv = load16(kr + e);
#pragma unroll
          for (int a4 = 0; a4 < 4; ++a4) {
            if (a4 < nh) {
#pragma unroll
              for (int u = 0; u < VN; u += 4) {
                const float4 qv = *reinterpret_cast<const float4*>(q + (h0 + a4) * d + e + u);
                acc[a4] = fmaf(qv.x, kv.get(u), acc[a4]);
                acc[a4] = fmaf(qv.y, kv.get(u + 1), acc[a4]);
                acc[a4] = fmaf(qv.z, kv.get(u + 2), acc[a4]);
                acc[a4] = fmaf(qv.w, kv.get(u + 3), acc[a4]);
              }
            }
          }
        }
      } else if (there) {
        for (int e = 0; e < d; ++e) {
          const float kv = to_f32(kr[e]);
#pragma unroll
          for (int a4 = 0; a4 < 4; ++a4)
            if (a4 < nh) acc[a4] = fmaf(q[(h0 + a4) * d + e], kv, acc[a4]);
        }
      }
#pragma unroll
      for (int a4 = 0; a4 < 4; ++a4) {
        if (a4 >= nh) continue;
        const int h = h0 + a4;
        float sc = -INFINITY;
        if (there) {
          sc = acc[a4] * scale;
          if (r1) sc -= r1[h] * log1pf(r2[h] * (float)(p - lo - j));
        }
        w[(size_t)h * max_keys + j] = sc;
      }
    }
  }
  __syncthreads();
  for (int h = warp; h < H; h += nwarps) {
    float* wh = w + (size_t)h * max_keys;
    float m = -INFINITY;
    for (int j = lane; j < n; j += 32) m = fmaxf(m, wh[j]);
    m = warp_max(m);
    float sum = 0.f;
    for (int j = lane; j < n; j += 32) {
      const float e = wh[j] == -INFINITY ? 0.f : expf(wh[j] - m);
      wh[j] = e;
      sum += e;
    }
    sum = warp_sum(sum);
    const float inv = sum > 0.f ? 1.0f / sum : 0.f;
    for (int j = lane; j < n; j += 32) wh[j] *= inv;
  }
  __syncthreads();
  if (talk) {
    // in place, a key's column of weights at a time: the thread that owns the key reads all heads' weights, then writes the mixed ones
    for (int j = threadIdx.x; j < n; j += blockDim.x) {
      float col[kMaxMixedHeads];
      for (int g = 0; g < H; ++g) col[g] = w[(size_t)g * max_keys + j];
      for (int h = 0; h < H; ++h) {
        float acc = 0.f;
        for (int g = 0; g < H; ++g) acc = fmaf(talk[h * H + g], col[g], acc);
        w[(size_t)h * max_keys + j] = acc;
      }
    }
    __syncthreads();
  }
  const float* use = w;
  // outputs: one (kv head, value element) pair per thread and turn, for up to four of the kv head's query heads at a
  // time, so that a value is fetched once for them; consecutive threads take consecutive elements
  for (int i = threadIdx.x; i < G * dv; i += blockDim.x) {
    const int c = i / dv, e = i % dv;
    const size_t head_off = (size_t)G * page_size * d + (size_t)c * page_size * dv + e;
    for (int h0 = c * group; h0 < (c + 1) * group; h0 += 4) {
      const int nh = min(4, (c + 1) * group - h0);
      const float* w0 = use + (size_t)h0 * max_keys;
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
      for (int j = 0; j < n; ++j) {                   // (eight keys per turn: their values are fetched side by side)
        // no branch in here: a key without a page (its weight is zero already) reads the first page's value
        const long long pg = page_at[j];
        const T raw = cache[(size_t)(pg < 0 ? 0 : pg) + head_off + (size_t)((lo + j) % page_size) * dv];
        const float v = pg < 0 ? 0.f : to_f32(raw);
#pragma unroll
        for (int a4 = 0; a4 < 4; ++a4)
          if (a4 < nh) acc[a4] = fmaf(w0[(size_t)a4 * max_keys + j], v, acc[a4]);
      }
#pragma unroll
      for (int a4 = 0; a4 < 4; ++a4)
        if (a4 < nh) out[(size_t)t * out_ld + column + (h0 + a4) * dv + e] = from_f32<T>(acc[a4] * out_scale);
    }
  }
}

template <typename T>
int kv_write_normed(void* cache, const void* qkv, const float* bias, const int* slots, int tokens, int H, int G, int d, int dv,
                    int page_size, long long num_slots, float eps, void* stream) {
  PTL_REQUIRE(tokens >= 0 && H > 0 && G > 0 && d > 0 && dv > 0 && page_size > 0 && eps >= 0.f,
              "kv_write_normed: bad sizes tokens=%d H=%d G=%d d=%d dv=%d page=%d", tokens, H, G, d, dv, page_size);
  if (tokens == 0) return 0;
  return launch_kernel("kv_write_normed", kv_write_normed_kernel<T>, dim3(tokens), dim3(128), 0, as_stream(stream), (T*)cache,
                       (const T*)qkv, bias, slots, H, G, d, dv, page_size, num_slots, eps);
}

template <typename T>
int chunk_attention(void* out, int out_ld, int column, const void* qkv, int q_ld, const float* q_bias, const void* cache,
                    const int* block_table, int table_width, const int* tok_req, const int* positions, int tokens, int H, int G,
                    int d, int dv, int page_size, float scale, int chunk, const float* r1, const float* r2, const float* talk,
                    int max_keys, int num_pages, float out_scale, void* stream) {
  PTL_REQUIRE(tokens >= 0 && H > 0 && G > 0 && H % G == 0 && d > 0 && dv > 0 && page_size > 0 && chunk >= 0 && max_keys > 0,
              "chunk_attention: bad sizes tokens=%d H=%d G=%d d=%d dv=%d page=%d chunk=%d keys=%d", tokens, H, G, d, dv, page_size,
              chunk, max_keys);
  PTL_REQUIRE((r1 == nullptr) == (r2 == nullptr), "chunk_attention: the distance bias needs both of its factors");
  PTL_REQUIRE(column >= 0 && column + H * dv <= out_ld && q_ld >= H * d, "chunk_attention: rows too short for the heads");
  if (tokens == 0) return 0;
  max_keys += max_keys & 1;            // the queries behind the page addresses start on a 16-byte boundary
  PTL_REQUIRE(!talk || H <= kMaxMixedHeads, "chunk_attention: weights of at most %d heads can be mixed, got %d", kMaxMixedHeads, H);
  const size_t smem = (size_t)max_keys * sizeof(long long) + ((size_t)H * d + (size_t)H * max_keys) * sizeof(float);
  PTL_REQUIRE(smem <= 200 * 1024, "chunk_attention: %d heads over %d keys do not fit the shared memory of a block (%zu bytes)", H,
              max_keys, smem);
  static SmemRaised raised = {};
  if (smem > 48 * 1024)
    if (int rc = raise_shared_memory("chunk_attention", chunk_attention_kernel<T>, 200 * 1024, raised)) return rc;
  const int vec_ok = d % Vec16<T>::N == 0 && dv % Vec16<T>::N == 0 && d % 4 == 0 && aligned16(cache);   // every key row starts on a 16-byte boundary
  return launch_kernel("chunk_attention", chunk_attention_kernel<T>, dim3(tokens), dim3(256), smem, as_stream(stream), (T*)out,
                       out_ld, column, (const T*)qkv, q_ld, q_bias, (const T*)cache, block_table, table_width, tok_req, positions,
                       H, G, d, dv, page_size, scale, chunk, r1, r2, talk, max_keys, num_pages, out_scale, vec_ok);
}

}  // namespace ptl

#define PTL_CHUNK_ATTENTION(SUFFIX, TYPE)                                                                                         \
  PTL_EXPORT int ptl_kv_write_normed##SUFFIX(void* cache, const void* qkv, const float* bias, const int* slots, int tokens, int H, \
                                             int G, int d, int dv, int page_size, long long num_slots, float eps, void* stream) { \
    return ptl::kv_write_normed<TYPE>(cache, qkv, bias, slots, tokens, H, G, d, dv, page_size, num_slots, eps, stream);            \
  }                                                                                                                               \
  PTL_EXPORT int ptl_chunk_attention##SUFFIX(void* out, int out_ld, int column, const void* qkv, int q_ld, const float* q_bias,    \
                                             const void* cache, const int* block_table, int table_width, const int* tok_req,      \
                                             const int* positions, int tokens, int H, int G, int d, int dv, int page_size,        \
                                             float scale, int chunk, const float* r1, const float* r2, const float* talk,         \
                                             int max_keys, int num_pages, float out_scale, void* stream) {                        \
    return ptl::chunk_attention<TYPE>(out, out_ld, column, qkv, q_ld, q_bias, cache, block_table, table_width, tok_req, positions, \
                                      tokens, H, G, d, dv, page_size, scale, chunk, r1, r2, talk, max_keys, num_pages, out_scale, \
                                      stream);                                                                                    \
  }
PTL_CHUNK_ATTENTION(_f32, float)
PTL_CHUNK_ATTENTION(_bf16, __nv_bfloat16)
