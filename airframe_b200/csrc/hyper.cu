// A residual stream kept in several copies ("streams") that every sublayer reads as one weighted sum and
// rewrites all at once (hyper-connections):
//   u      = sum_s in[s] x_s                          what the sublayer's norm reads
//   x'_t   = sum_s mix[s][t] x_s + out[t] (ls * y)    every stream from the old ones and the sublayer's result y
// x is float32 [tokens, streams, width]; y arrives as one or two terms (tensors of the compute dtype or of
// float32, or float32 partial sums that are added in index order), optionally times a per-channel layer scale.
//   hc_read     u and its RMS norm (offset + w) in the compute dtype
//   hc_write    the rewrite, and in the same pass the next sublayer's u and norm
//   stream_copy every stream = the embedding's row;  stream_sum  the sum of the streams
// All sums are 32-bit.  One block per token; a thread owns groups of VEC neighbouring channels.
#include "common.cuh"

#define AF_HC_MAX 16

struct AfHcTerm {
  const void* p;
  int dtype, parts;
  float scale;
};

template <int VEC>
__device__ __forceinline__ void hc_term_add(float* acc, const AfHcTerm& t, size_t part_stride, size_t at) {
  if (t.p == nullptr) return;
  if (t.dtype == AF_BF16) {
    const __nv_bfloat16* b = static_cast<const __nv_bfloat16*>(t.p) + at;
    if (VEC == 4) {
      const uint2 raw = *reinterpret_cast<const uint2*>(b);
      acc[0] += t.scale * __uint_as_float(raw.x << 16);
      acc[1 % VEC] += t.scale * __uint_as_float(raw.x & 0xffff0000u);
      acc[2 % VEC] += t.scale * __uint_as_float(raw.y << 16);
      acc[3 % VEC] += t.scale * __uint_as_float(raw.y & 0xffff0000u);
    } else {
      acc[0] += t.scale * __bfloat162float(b[0]);
    }
    return;
  }
  const float* f = static_cast<const float*>(t.p) + at;
  float v[VEC];
#pragma unroll
  for (int u = 0; u < VEC; ++u) v[u] = 0.f;
  for (int s = 0; s < t.parts; ++s) {
    if (VEC == 4) {
      const float4 q = *reinterpret_cast<const float4*>(f + (size_t)s * part_stride);
      v[0] += q.x, v[1 % VEC] += q.y, v[2 % VEC] += q.z, v[3 % VEC] += q.w;
    } else {
      v[0] += f[(size_t)s * part_stride];
    }
  }
#pragma unroll
  for (int u = 0; u < VEC; ++u) acc[u] += t.scale * v[u];
}

template <int VEC>
__device__ __forceinline__ void hc_load(float* v, const float* p) {
  if (VEC == 4) {
    const float4 q = *reinterpret_cast<const float4*>(p);
    v[0] = q.x, v[1 % VEC] = q.y, v[2 % VEC] = q.z, v[3 % VEC] = q.w;
  } else {
    v[0] = p[0];
  }
}

template <int VEC>
__device__ __forceinline__ void hc_store(float* p, const float* v) {
  if (VEC == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1 % VEC], v[2 % VEC], v[3 % VEC]);
  else p[0] = v[0];
}

// y[t] = norm(sum_s in[s] x[t][s]) (offset + w)
template <typename TY, int VEC>
__global__ void __launch_bounds__(640)
hc_read_kernel(TY* __restrict__ y, const float* __restrict__ x, const float* __restrict__ in_w,
               const float* __restrict__ w, float eps, float offset, int S, int W) {
  pdl_launch_dependents();
  extern __shared__ float row[];
  __shared__ float scratch[33];
  __shared__ float cin[AF_HC_MAX];
  if (threadIdx.x < S) cin[threadIdx.x] = in_w[threadIdx.x];
  pdl_wait();
  x = pdl_fresh(x);
  __syncthreads();
  const size_t t = blockIdx.x;
  const float* xt = x + t * S * W;
  float ss = 0.f;
  for (int i = threadIdx.x * VEC; i < W; i += blockDim.x * VEC) {
    float u[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) u[e] = 0.f;
    for (int s = 0; s < S; ++s) {
      float v[VEC];
      hc_load<VEC>(v, xt + (size_t)s * W + i);
#pragma unroll
      for (int e = 0; e < VEC; ++e) u[e] = fmaf(cin[s], v[e], u[e]);
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      row[i + e] = u[e];
      ss += u[e] * u[e];
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) y[t * W + i] = from_f32<TY>(row[i] * inv * (offset + w[i]));
}

// x[t][.] rewritten from the sublayer's result; with y: the next sublayer's norm(sum_s in_next[s] x'[t][s]) (offset + w_next)
// SMAX: the streams a thread has registers for (2, 4, 8 or 16: the smallest that holds S; with up to four streams two
// blocks share an SM, so that one block's loads run under another's reduction; sixteen want narrow blocks).
template <typename TY, int VEC, int SMAX>
__global__ void __launch_bounds__(SMAX <= 4 ? 512 : SMAX <= 8 ? 640 : 256, SMAX <= 4 ? 2 : 1)
hc_write_kernel(float* __restrict__ x, AfHcTerm a, AfHcTerm b, size_t part_stride, const float* __restrict__ ls,
                const float* __restrict__ mix, const float* __restrict__ out_w, const float* __restrict__ in_next,
                const float* __restrict__ w_next, float eps, float offset, TY* __restrict__ y, int S, int W) {
  pdl_launch_dependents();
  extern __shared__ float row[];
  __shared__ float scratch[33];
  __shared__ float cmix[AF_HC_MAX * AF_HC_MAX], cout[AF_HC_MAX], cin[AF_HC_MAX];
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) cmix[i] = mix[i];      // (a block may have fewer threads than S * S)
  if (threadIdx.x < S) {
    cout[threadIdx.x] = out_w[threadIdx.x];
    cin[threadIdx.x] = in_next != nullptr ? in_next[threadIdx.x] : 0.f;
  }
  pdl_wait();
  x = pdl_fresh(x);
  a.p = pdl_fresh(a.p);
  b.p = pdl_fresh(b.p);
  __syncthreads();
  const size_t t = blockIdx.x;
  float* xt = x + t * S * W;
  float ss = 0.f;
  for (int i = threadIdx.x * VEC; i < W; i += blockDim.x * VEC) {
    float yv[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) yv[e] = 0.f;
    hc_term_add<VEC>(yv, a, part_stride, t * W + i);
    hc_term_add<VEC>(yv, b, part_stride, t * W + i);
    if (ls != nullptr) {
      float l[VEC];
      hc_load<VEC>(l, ls + i);
#pragma unroll
      for (int e = 0; e < VEC; ++e) yv[e] *= l[e];
    }
    float xs[SMAX][VEC];
#pragma unroll
    for (int s = 0; s < SMAX; ++s)
      if (s < S) hc_load<VEC>(xs[s], xt + (size_t)s * W + i);
    float u[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) u[e] = 0.f;
#pragma unroll
    for (int to = 0; to < SMAX; ++to) {
      if (to >= S) continue;
      float nv[VEC];
#pragma unroll
      for (int e = 0; e < VEC; ++e) nv[e] = 0.f;
#pragma unroll
      for (int s = 0; s < SMAX; ++s) {
        if (s >= S) continue;
        const float c = cmix[s * S + to];
#pragma unroll
        for (int e = 0; e < VEC; ++e) nv[e] = fmaf(c, xs[s][e], nv[e]);
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        nv[e] = fmaf(cout[to], yv[e], nv[e]);
        u[e] = fmaf(cin[to], nv[e], u[e]);
      }
      hc_store<VEC>(xt + (size_t)to * W + i, nv);
    }
    if (y != nullptr) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        row[i + e] = u[e];
        ss += u[e] * u[e];
      }
    }
  }
  if (y == nullptr) return;
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) y[t * W + i] = from_f32<TY>(row[i] * inv * (offset + w_next[i]));
}

__global__ void __launch_bounds__(256)
stream_copy_kernel(float* __restrict__ x, const float* __restrict__ e, int S, int W) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t t = blockIdx.x;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = e[t * W + i];
    for (int s = 0; s < S; ++s) x[(t * S + s) * W + i] = v;
  }
}

__global__ void __launch_bounds__(256)
stream_sum_kernel(float* __restrict__ out, const float* __restrict__ x, int S, int W) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t t = blockIdx.x;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < S; ++s) v += x[(t * S + s) * W + i];
    out[t * W + i] = v;
  }
}

// Threads of a token's block: as many as give every thread the same number of channel groups, up to `most` (all loads of a
// thread's groups are in flight at once).
static int hc_threads(int W, int vec, int most = 640) {
  const int groups = (W + vec - 1) / vec;
  const int iters = (groups + most - 1) / most;
  int th = (((groups + iters - 1) / iters + 31) / 32) * 32;
  return th < 32 ? 32 : th > most ? most : th;
}

AF_EXPORT int af_hc_read(void* y, int y_dtype, const float* x, const float* in_w, const float* w, float eps, float offset,
                         int n_tokens, int S, int W, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && S >= 1 && S <= AF_HC_MAX && W > 0, "af_hc_read: up to %d streams", AF_HC_MAX);
  AF_REQUIRE((size_t)W * sizeof(float) <= 48 * 1024, "af_hc_read: rows of up to 12288 values");
  const bool vec = W % 4 == 0 && ((uintptr_t)x & 15) == 0;
  const size_t smem = (size_t)W * sizeof(float);
  if (vec) {
    AF_DISPATCH_DTYPE(y_dtype, TY, af_launch(hc_read_kernel<TY, 4>, dim3(n_tokens), dim3(hc_threads(W, 4)), smem, stream,
                                             (TY*)y, x, in_w, w, eps, offset, S, W));
  } else {
    AF_DISPATCH_DTYPE(y_dtype, TY, af_launch(hc_read_kernel<TY, 1>, dim3(n_tokens), dim3(hc_threads(W, 1)), smem, stream,
                                             (TY*)y, x, in_w, w, eps, offset, S, W));
  }
  AF_CHECK_LAUNCH("af_hc_read");
}

// a, b: the terms of the sublayer's result ([n_tokens, W] of a_dtype, or a_parts float partial sums [parts, n_tokens, W]);
// b may be null.  ls: the layer scale [W] or null.  y null: no next sublayer is read.
AF_EXPORT int af_hc_write(float* x, const void* a, int a_dtype, int a_parts, float scale_a, const void* b, int b_dtype,
                          int b_parts, float scale_b, const float* ls, const float* mix, const float* out_w,
                          const float* in_next, const float* w_next, float eps, float offset, void* y, int y_dtype,
                          int n_tokens, int S, int W, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && S >= 1 && S <= AF_HC_MAX && W > 0 && a != nullptr && a_parts >= 1 && b_parts >= 1,
             "af_hc_write: up to %d streams, at least one term", AF_HC_MAX);
  AF_REQUIRE((a_dtype == AF_F32 || (a_dtype == AF_BF16 && a_parts == 1)) &&
             (b == nullptr || b_dtype == AF_F32 || (b_dtype == AF_BF16 && b_parts == 1)),
             "af_hc_write: partial sums are float");
  AF_REQUIRE(y == nullptr || (in_next != nullptr && w_next != nullptr), "af_hc_write: the next read needs its weights");
  AF_REQUIRE((size_t)W * sizeof(float) <= 48 * 1024, "af_hc_write: rows of up to 12288 values");
  const AfHcTerm ta{a, a_dtype, a_parts, scale_a}, tb{b, b_dtype, b_parts, scale_b};
  const size_t part_stride = (size_t)n_tokens * W;
  const bool vec = W % 4 == 0 && (((uintptr_t)x | (uintptr_t)a | (uintptr_t)b | (uintptr_t)ls) & 15) == 0;
  const size_t smem = y != nullptr ? (size_t)W * sizeof(float) : 0;
#define AF_HC_LAUNCH(VEC_, SMAX_)                                                                                      \
  AF_DISPATCH_DTYPE(y_dtype, TY,                                                                                       \
                    af_launch(hc_write_kernel<TY, VEC_, SMAX_>, dim3(n_tokens), dim3(hc_threads(W, VEC_, SMAX_ <= 4 ? 512 : SMAX_ <= 8 ? 640 : 256)), smem, \
                              stream, x, ta, tb, part_stride, ls, mix, out_w, in_next, w_next, eps, offset, (TY*)y, S, W))
  // few tokens (a decode step): the variant with registers for eight streams, whose blocks may be wide enough to
  // have all of a row's loads in flight at once; many tokens: the smallest that holds S, two blocks an SM
  const bool few = n_tokens < 512;
  if (vec) {
    if (S <= 2 && !few) AF_HC_LAUNCH(4, 2);
    else if (S <= 4 && !few) AF_HC_LAUNCH(4, 4);
    else if (S <= 8) AF_HC_LAUNCH(4, 8);
    else AF_HC_LAUNCH(4, 16);
  } else {
    if (S <= 2 && !few) AF_HC_LAUNCH(1, 2);
    else if (S <= 4 && !few) AF_HC_LAUNCH(1, 4);
    else if (S <= 8) AF_HC_LAUNCH(1, 8);
    else AF_HC_LAUNCH(1, 16);
  }
#undef AF_HC_LAUNCH
  AF_CHECK_LAUNCH("af_hc_write");
}

AF_EXPORT int af_stream_copy(float* x, const float* e, int n_tokens, int S, int W, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && S >= 1 && W > 0, "af_stream_copy: bad sizes");
  af_launch(stream_copy_kernel, dim3(n_tokens), dim3(256), 0, stream, x, e, S, W);
  AF_CHECK_LAUNCH("af_stream_copy");
}

AF_EXPORT int af_stream_sum(float* out, const float* x, int n_tokens, int S, int W, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && S >= 1 && W > 0, "af_stream_sum: bad sizes");
  af_launch(stream_sum_kernel, dim3(n_tokens), dim3(256), 0, stream, out, x, S, W);
  AF_CHECK_LAUNCH("af_stream_sum");
}
