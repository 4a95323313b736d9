// A routed feed-forward (mixture of experts) without a word read back by the host:
//   expert_route   per token the router's logits in 32 bits, a score per expert (the sigmoid of its logit), the `top`
//                  experts with the largest scores (equal scores: the lower index) and their scores (optionally: a
//                  correction added to the scores for the choice only, a choice among the best groups of experts,
//                  weights divided by their sum and scaled); also the
//                  sigmoid of one more row of the router matrix when there is one (the gate of a shared expert);
//   expert_plan    the (token, choice) pairs sorted by expert: a permutation, and a table of tiles of up to 32
//                  pairs of one expert each;
//   expert_rows    a tile's rows times its expert's matrices on the CUDA cores, 32-bit sums in index order:
//                  either gate and up with the activation behind them, or down.
// The order of the pairs of an expert depends on the order in which blocks arrive, but every row of a tile is
// worked out by itself, so no result depends on it.
#include "common.cuh"

#define AF_EX_TM 32
#define AF_EX_TN 64
#define AF_EX_TK 32

// ---------------------------------------------------------------- the router

template <typename TX>
__device__ __forceinline__ void load4_f32(float* v, const TX* p);
template <>
__device__ __forceinline__ void load4_f32<float>(float* v, const float* p) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
}
template <>
__device__ __forceinline__ void load4_f32<__nv_bfloat16>(float* v, const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  v[0] = __uint_as_float(raw.x << 16), v[1] = __uint_as_float(raw.x & 0xffff0000u);
  v[2] = __uint_as_float(raw.y << 16), v[3] = __uint_as_float(raw.y & 0xffff0000u);
}

// Scores first, the choice behind them.  A warp of the scores' kernel takes one row of the router (an expert, or
// the shared expert's gate) and TM tokens, and adds a token's products in one fixed order whatever TM is, so that a
// prompt and a decode step choose alike; the warps of a block share their tokens.  scores: [tokens, rows].
template <typename TX, int TM>
__global__ void __launch_bounds__(256)
expert_score_kernel(float* __restrict__ scores, const TX* __restrict__ h, const float* __restrict__ router, int n_tokens,
                    int hidden, int rows) {
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long job = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  const long long groups = (n_tokens + TM - 1) / TM;
  if (job >= groups * rows) return;
  const int t0 = (int)(job / rows) * TM, e = (int)(job % rows);
  const float* w = router + (size_t)e * hidden;
  const bool vec = hidden % 4 == 0 && (((uintptr_t)h | (uintptr_t)router) & 15) == 0;
  pdl_wait();
  h = pdl_fresh(h);
  float z[TM];
  if (vec) {                                        // four values a lane and load, four loads in flight
    float zz[TM][4];
#pragma unroll
    for (int m = 0; m < TM; ++m) zz[m][0] = zz[m][1] = zz[m][2] = zz[m][3] = 0.f;
    for (int i0 = lane * 4; i0 < hidden; i0 += 512) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * 128;
        if (i < hidden) {
          const float4 wv = *reinterpret_cast<const float4*>(w + i);
#pragma unroll
          for (int m = 0; m < TM; ++m) {
            if (t0 + m >= n_tokens) continue;
            float xv[4];
            load4_f32<TX>(xv, h + (size_t)(t0 + m) * hidden + i);
            zz[m][u] = fmaf(wv.x, xv[0], fmaf(wv.y, xv[1], fmaf(wv.z, xv[2], fmaf(wv.w, xv[3], zz[m][u]))));
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < TM; ++m) z[m] = (zz[m][0] + zz[m][1]) + (zz[m][2] + zz[m][3]);
  } else {
#pragma unroll
    for (int m = 0; m < TM; ++m) {
      z[m] = 0.f;
      if (t0 + m >= n_tokens) continue;
      const TX* x = h + (size_t)(t0 + m) * hidden;
      for (int i = lane; i < hidden; i += 32) z[m] = fmaf(w[i], to_f32<TX>(x[i]), z[m]);
    }
  }
#pragma unroll
  for (int m = 0; m < TM; ++m) {
    const float zs = warp_sum(z[m]);
    if (lane == 0 && t0 + m < n_tokens) scores[(size_t)(t0 + m) * rows + e] = 1.f / (1.f + expf(-zs));
  }
}

// A warp a token: the `top` largest choice scores in turn (equal scores: the lower index), each struck out once
// chosen.  The choice score is the score plus `correction[e]` (none: the score); the weight is always the score
// itself.  With `groups` > 1 the experts form that many equal groups of neighbours, a group's score is the sum of its
// two largest choice scores (of its only one, in groups of one), and only experts of the `keep` best groups (equal
// scores: the lower group) can be chosen.  With `normalise` the chosen weights are divided by their sum + 1e-20;
// all weights are multiplied by `out_scale`.
__global__ void __launch_bounds__(128)
expert_choose_kernel(int* __restrict__ ids, float* __restrict__ wts, float* __restrict__ shared_gate,
                     const float* __restrict__ scores, const float* __restrict__ correction, int n_tokens,
                     int n_experts, int rows, int top, int groups, int keep, int normalise, float out_scale) {
  pdl_launch_dependents();
  extern __shared__ float score_all[];              // a warp: n_experts choice scores, n_experts scores, `groups` group scores
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  pdl_wait();
  if (t >= n_tokens) return;
  scores = pdl_fresh(scores);
  float* choice = score_all + (size_t)warp * (2 * n_experts + groups);
  float* score = choice + n_experts;
  float* gscore = score + n_experts;
  const float OUT = -3.0e38f;                       // an expert of a group that is not kept (it still beats a struck one)
  const float STRUCK = -INFINITY;
  for (int e = lane; e < n_experts; e += 32) {
    const float sc = scores[(size_t)t * rows + e];
    score[e] = sc;
    choice[e] = sc + (correction != nullptr ? correction[e] : 0.f);
  }
  if (shared_gate != nullptr && lane == 0) shared_gate[t] = scores[(size_t)t * rows + n_experts];
  __syncwarp();
  if (groups > 1 && keep < groups) {
    const int per = n_experts / groups;
    for (int g = lane; g < groups; g += 32) {
      float a = STRUCK, b = STRUCK;                 // the two largest of the group
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float c = choice[e];
        if (c > a) b = a, a = c;
        else if (c > b) b = c;
      }
      gscore[g] = per > 1 ? a + b : a;
    }
    __syncwarp();
    for (int k = 0; k < keep; ++k) {                // the best groups in turn, marked by +infinity
      float best = STRUCK;
      int at = groups;
      for (int g = lane; g < groups; g += 32)
        if (gscore[g] != INFINITY && gscore[g] > best) best = gscore[g], at = g;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (ob > best || (ob == best && oa < at)) best = ob, at = oa;
      }
      if (lane == 0 && at < groups) gscore[at] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < n_experts; e += 32)
      if (gscore[e / per] != INFINITY) choice[e] = OUT;
    __syncwarp();
  }
  float total = 0.f;                                // (lane 0's)
  for (int k = 0; k < top; ++k) {
    float best = STRUCK;
    int at = n_experts;
    for (int e = lane; e < n_experts; e += 32)
      if (choice[e] > best) best = choice[e], at = e; // (ascending e: the lower index wins among equals)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) best = ob, at = oa;
    }
    if (lane == 0) {
      if (at >= n_experts) at = 0;                  // (cannot be: top <= n_experts, and every expert's choice score is finite)
      ids[(size_t)t * top + k] = at;
      wts[(size_t)t * top + k] = score[at];
      total += score[at];
      choice[at] = STRUCK;
    }
    __syncwarp();
  }
  if (lane == 0) {
    const float f = normalise ? out_scale / (total + 1e-20f) : out_scale;
    if (normalise || out_scale != 1.f)
      for (int k = 0; k < top; ++k) wts[(size_t)t * top + k] *= f;
  }
}

// scores: room for n_tokens x (n_experts + 1) floats.
AF_EXPORT int af_expert_route(int* ids, float* wts, float* shared_gate, float* scores, const void* h, int h_dtype,
                              const float* router, int n_tokens, int hidden, int n_experts, int top,
                              const float* correction, int groups, int keep, int normalise, float out_scale,
                              cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && hidden > 0 && n_experts > 0 && top >= 1 && top <= n_experts && scores != nullptr,
             "af_expert_route: %d of %d experts", top, n_experts);
  AF_REQUIRE(n_experts <= 8192, "af_expert_route: up to 8192 experts");
  if (groups < 1) groups = 1;
  AF_REQUIRE(n_experts % groups == 0 && keep >= 1 && keep <= groups && (long long)keep * (n_experts / groups) >= top,
             "af_expert_route: %d experts in %d groups of which %d are kept cannot give %d choices", n_experts, groups,
             keep, top);
  const int rows = n_experts + (shared_gate != nullptr ? 1 : 0);
  // a prompt: four tokens a warp (a row of the router is read once for them); few tokens: a warp each
  const int tm = n_tokens >= 256 ? 4 : 1;
  const long long jobs = (long long)((n_tokens + tm - 1) / tm) * rows;
  const long long blocks = (jobs + 7) / 8;
  AF_REQUIRE(blocks < (1ll << 31), "af_expert_route: too many tokens");
  if (tm == 4) {
    AF_DISPATCH_DTYPE(h_dtype, TX,
                      af_launch(expert_score_kernel<TX, 4>, dim3((unsigned)blocks), dim3(256), 0, stream, scores,
                                (const TX*)h, router, n_tokens, hidden, rows));
  } else {
    AF_DISPATCH_DTYPE(h_dtype, TX,
                      af_launch(expert_score_kernel<TX, 1>, dim3((unsigned)blocks), dim3(256), 0, stream, scores,
                                (const TX*)h, router, n_tokens, hidden, rows));
  }
  AF_COUNT_LAUNCH("af_expert_route");
  const int warps = n_experts <= 1024 ? 4 : 1;
  af_launch(expert_choose_kernel, dim3((n_tokens + warps - 1) / warps), dim3(32 * warps),
            (size_t)warps * (2 * n_experts + groups) * sizeof(float), stream, ids, wts, shared_gate, (const float*)scores,
            correction, n_tokens, n_experts, rows, top, groups, keep, normalise, out_scale);
  AF_CHECK_LAUNCH("af_expert_route");
}

// ---------------------------------------------------------------- pairs by expert

// One block.  plan: [0] tiles in use; then per tile (expert, first sorted row, rows).  perm[sorted row] = pair.
__global__ void __launch_bounds__(1024)
expert_plan_kernel(int* __restrict__ perm, int* __restrict__ plan, const int* __restrict__ ids, int n_pairs,
                   int n_experts, int max_tiles, int tile) {
  pdl_launch_dependents();
  extern __shared__ int sh[];                       // count[E], first[E], cursor[E]
  int* count = sh;
  int* first = sh + n_experts;
  int* cursor = sh + 2 * n_experts;
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) count[e] = 0, cursor[e] = 0;
  __syncthreads();
  pdl_wait();
  ids = pdl_fresh(ids);
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = ids[p];
    if (AF_INDEX_OK(e >= 0 && e < n_experts, e)) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int rows = 0, tiles = 0;
    for (int e = 0; e < n_experts; ++e) {
      first[e] = rows;
      // an expert's rows in as few tiles as hold them, of equal size (a last tile of a few rows costs a wide
      // tile's set-up for nothing)
      const int n_t = (count[e] + tile - 1) / tile;
      const int per = n_t > 0 ? (count[e] + n_t - 1) / n_t : 0;
      for (int r = 0; r < count[e] && tiles < max_tiles; r += per, ++tiles) {
        plan[1 + 3 * tiles] = e;
        plan[2 + 3 * tiles] = rows + r;
        plan[3 + 3 * tiles] = min(per, count[e] - r);
      }
      rows += count[e];
    }
    plan[0] = tiles;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < n_experts) perm[first[e] + atomicAdd(&cursor[e], 1)] = p;
  }
}

AF_EXPORT int af_expert_plan(int* perm, int* plan, const int* ids, int n_pairs, int n_experts, int max_tiles,
                             int tile, cudaStream_t stream) {
  if (n_pairs == 0) return 0;
  AF_REQUIRE(n_pairs > 0 && n_experts > 0 && n_experts <= 4096 && tile > 0, "af_expert_plan: bad sizes");
  // (every expert may end on a tile that is not full)
  AF_REQUIRE(max_tiles >= n_pairs / tile + n_experts || max_tiles >= n_pairs,
             "af_expert_plan: room for %d tiles is too little", max_tiles);
  af_launch(expert_plan_kernel, dim3(1), dim3(1024), (size_t)3 * n_experts * sizeof(int), stream, perm, plan, ids,
            n_pairs, n_experts, max_tiles, tile);
  AF_CHECK_LAUNCH("af_expert_plan");
}

// ---------------------------------------------------------------- the tokens' rows in sorted order

// out[sorted row] = x[perm[sorted row] / top]: the rows a tensor-core product fetches tile by tile.
template <typename T>
__global__ void __launch_bounds__(256)
expert_gather_kernel(T* __restrict__ out, const T* __restrict__ x, const int* __restrict__ perm, int n_rows, int top,
                     int H) {
  pdl_launch_dependents();
  pdl_wait();
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * warps + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  const int pair = __ldcg(perm + r);
  if (!AF_INDEX_OK(pair >= 0 && pair < n_rows, pair)) return;
  const T* src = x + (size_t)(pair / top) * H;
  T* dst = out + (size_t)r * H;
  if ((H * sizeof(T)) % 16 == 0) {
    const int n16 = H * sizeof(T) / 16;
    for (int i = lane; i < n16; i += 32) reinterpret_cast<int4*>(dst)[i] = __ldcg(reinterpret_cast<const int4*>(src) + i);
  } else {
    for (int i = lane; i < H; i += 32) dst[i] = src[i];
  }
}

AF_EXPORT int af_expert_gather(void* out, const void* x, int dtype, const int* perm, int n_rows, int top, int H,
                               cudaStream_t stream) {
  if (n_rows == 0) return 0;
  AF_REQUIRE(n_rows > 0 && top >= 1 && H > 0 && perm != nullptr, "af_expert_gather: bad sizes");
  AF_REQUIRE(((uintptr_t)out & 15) == 0 && ((uintptr_t)x & 15) == 0, "af_expert_gather: rows must be 16-byte aligned");
  AF_DISPATCH_DTYPE(dtype, T,
                    af_launch(expert_gather_kernel<T>, dim3((n_rows + 7) / 8), dim3(256), 0, stream, (T*)out,
                              (const T*)x, perm, n_rows, top, H));
  AF_CHECK_LAUNCH("af_expert_gather");
}

// ---------------------------------------------------------------- a tile's rows times its expert's matrices

// The activation of these experts: g = min(g, limit), u = clamp(u, -limit, limit), g sigmoid(1.702 g) (u + 1).
__device__ __forceinline__ float clamped_glu(float g, float u, float limit) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.f + expf(-1.702f * g)) * (u + 1.f);
}

// DUAL: out[sorted row][n] = act(s (x . w0[e][n]), s (x . w1[e][n])) * post, x the row of `a` that the pair's
//       token names, s the pair's weight (a weight on an expert's input goes through its products, which have no
//       bias), post the token's `scale_out` (1 without); out of the compute dtype, rows of N values.
// MODE 2: out[sorted row][n] = gelu(x . w0[e][n]) * s * post with the exact (erf) GELU: an expert of one matrix, whose
//       weight stands behind the activation.
// else: out[(choice, token)][n] = a[sorted row] . w0[e][n] as floats: [top][tokens][N], partial sums that the
//       residual kernel adds.
// Without a plan (plan == nullptr) there is one expert and the rows are the tokens in order.
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
expert_rows_kernel(void* __restrict__ out_, const T* __restrict__ a, const T* __restrict__ w0, const T* __restrict__ w1,
                   const int* __restrict__ perm, const int* __restrict__ plan, const float* __restrict__ pair_weight,
                   const float* __restrict__ scale_out, int n_rows, int n_tokens, int top, int N, int K, float limit) {
  pdl_launch_dependents();
  constexpr bool DUAL = MODE == 1;                  // gate and up with the clamped activation
  constexpr bool MID = MODE != 0;                   // rows out in sorted order, of the compute dtype (MODE 2: one matrix, exact GELU)
  __shared__ float as[AF_EX_TM][AF_EX_TK];
  __shared__ float w0s[AF_EX_TN][AF_EX_TK + 1];
  __shared__ float w1s[DUAL ? AF_EX_TN : 1][AF_EX_TK + 1];
  __shared__ int src_row[AF_EX_TM];                 // the row of `a` a tile row reads (-1: none)
  __shared__ int pair_of[AF_EX_TM];
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  const int n0 = blockIdx.y * AF_EX_TN;
  pdl_wait();
  plan = pdl_fresh(plan);
  perm = pdl_fresh(perm);
  a = pdl_fresh(a);
  int expert = 0, row0 = blockIdx.x * AF_EX_TM, rows = min(AF_EX_TM, n_rows - row0);
  if (plan != nullptr) {
    if ((int)blockIdx.x >= plan[0]) return;
    expert = plan[1 + 3 * blockIdx.x], row0 = plan[2 + 3 * blockIdx.x], rows = plan[3 + 3 * blockIdx.x];
  }
  if (rows <= 0) return;
  if (threadIdx.x < AF_EX_TM) {
    const int m = threadIdx.x;
    int pair = -1;
    if (m < rows) pair = perm != nullptr ? perm[row0 + m] : row0 + m;
    pair_of[m] = pair;
    src_row[m] = pair < 0 ? -1 : (MID ? pair / top : row0 + m);
  }
  __syncthreads();
  const T* w0e = w0 + (size_t)expert * N * K;
  const T* w1e = DUAL ? w1 + (size_t)expert * N * K : nullptr;
  float acc0[AF_EX_TM / 4], acc1[AF_EX_TM / 4];
#pragma unroll
  for (int m = 0; m < AF_EX_TM / 4; ++m) acc0[m] = acc1[m] = 0.f;
  for (int k0 = 0; k0 < K; k0 += AF_EX_TK) {
    for (int e = threadIdx.x; e < AF_EX_TM * AF_EX_TK; e += 256) {
      const int m = e / AF_EX_TK, k = e % AF_EX_TK;
      const int r = src_row[m];
      as[m][k] = (r >= 0 && k0 + k < K) ? to_f32<T>(a[(size_t)r * K + k0 + k]) : 0.f;
    }
    for (int e = threadIdx.x; e < AF_EX_TN * AF_EX_TK; e += 256) {
      const int n = e / AF_EX_TK, k = e % AF_EX_TK;
      const bool in = n0 + n < N && k0 + k < K;
      w0s[n][k] = in ? to_f32<T>(w0e[(size_t)(n0 + n) * K + k0 + k]) : 0.f;
      if (DUAL) w1s[n][k] = in ? to_f32<T>(w1e[(size_t)(n0 + n) * K + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < AF_EX_TK; ++k) {
      const float p = w0s[tx][k];
      const float q = DUAL ? w1s[tx][k] : 0.f;
#pragma unroll
      for (int m = 0; m < AF_EX_TM / 4; ++m) {
        const float v = as[ty + 4 * m][k];
        acc0[m] = fmaf(p, v, acc0[m]);
        if (DUAL) acc1[m] = fmaf(q, v, acc1[m]);
      }
    }
    __syncthreads();
  }
  const int n = n0 + tx;
  if (n >= N) return;
#pragma unroll
  for (int m = 0; m < AF_EX_TM / 4; ++m) {
    const int row = ty + 4 * m;
    const int pair = pair_of[row];
    if (pair < 0) continue;
    if (MID) {
      const float s = pair_weight != nullptr ? pair_weight[pair] : 1.f;
      const float post = scale_out != nullptr ? scale_out[pair / top] : 1.f;
      const float val = DUAL ? clamped_glu(s * acc0[m], s * acc1[m], limit) * post
                             : 0.5f * acc0[m] * (1.f + erff(acc0[m] * 0.70710678118654752f)) * s * post;
      static_cast<T*>(out_)[(size_t)(row0 + row) * N + n] = from_f32<T>(val);
    } else {
      const int token = pair / top, choice = pair % top;
      static_cast<float*>(out_)[((size_t)choice * n_tokens + token) * N + n] = acc0[m];
    }
  }
}

AF_EXPORT int af_expert_rows(void* out, const void* a, const void* w0, const void* w1, int dtype, const int* perm,
                             const int* plan, const float* pair_weight, const float* scale_out, int n_rows,
                             int n_tokens, int top, int max_tiles, int N, int K, float limit, int act,
                             cudaStream_t stream) {
  if (n_rows == 0) return 0;
  AF_REQUIRE(n_rows > 0 && n_tokens > 0 && top >= 1 && N > 0 && K > 0, "af_expert_rows: bad sizes");
  AF_REQUIRE((plan == nullptr) == (perm == nullptr), "af_expert_rows: a plan and its permutation, or neither");
  AF_REQUIRE(n_rows == n_tokens * top, "af_expert_rows: %d rows for %d tokens with %d choices", n_rows, n_tokens, top);
  const int tiles = plan != nullptr ? max_tiles : (n_rows + AF_EX_TM - 1) / AF_EX_TM;
  AF_REQUIRE(tiles > 0, "af_expert_rows: no tiles");
  const dim3 grid(tiles, (N + AF_EX_TN - 1) / AF_EX_TN);
  AF_REQUIRE(grid.y < 65536, "af_expert_rows: too many outputs");
  if (w1 != nullptr) {
    AF_DISPATCH_DTYPE(dtype, T,
                      af_launch(expert_rows_kernel<T, 1>, grid, dim3(256), 0, stream, out, (const T*)a, (const T*)w0,
                                (const T*)w1, perm, plan, pair_weight, scale_out, n_rows, n_tokens, top, N, K, limit));
  } else if (act == 1) {
    AF_DISPATCH_DTYPE(dtype, T,
                      af_launch(expert_rows_kernel<T, 2>, grid, dim3(256), 0, stream, out, (const T*)a, (const T*)w0,
                                (const T*)nullptr, perm, plan, pair_weight, scale_out, n_rows, n_tokens, top, N, K, limit));
  } else {
    AF_DISPATCH_DTYPE(dtype, T,
                      af_launch(expert_rows_kernel<T, 0>, grid, dim3(256), 0, stream, out, (const T*)a, (const T*)w0,
                                (const T*)nullptr, perm, plan, pair_weight, scale_out, n_rows, n_tokens, top, N, K, limit));
  }
  AF_CHECK_LAUNCH("af_expert_rows");
}
