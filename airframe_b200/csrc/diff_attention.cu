// What stands around the attention kernels in differential attention: every query head and every key/value head
// carries two score maps over the same values, whose outputs a1 and a2 are joined as a1 - lambda a2.
//
//   conv_pack     from the float32 projection rows [q | k | v] (+ bias): a short causal convolution over time on
//                 every channel (taps from the step's own rows and, before them, from the sequence's history of
//                 projected values), the query temperature 1 + coef ln(floor((p + 1) / every) + 1), and the packing
//                 for the attention kernels: the two maps become heads of their own.  Query head h (group g = h / rep,
//                 j = h % rep, rep query heads a key/value head) with map m goes to head g (2 rep) + m rep + j; key
//                 head g with map m to head 2 g + m; value head g to heads 2 g and 2 g + 1.  So the grouped attention
//                 kernels, which give query head i the key/value head i / rep, need no change.  k and v also go to
//                 each token's row of its cache page.
//   conv_history  the sequence's last taps - 1 projected values (bias in, before the convolution), kept per slot.
//   diff_join     per head: o = a1 - lambda a2, o / sqrt(mean(o^2) + eps) * post, times sigmoid(gate); and a
//                 column of ones behind the heads (the output projection's bias rides as one more weight column).
// Everything here is 32-bit up to the rounding of what is written in the compute dtype.
#include "common.cuh"

struct AfConvArgs {
  const float* proj;           // [tokens, ld]: q at 0, k at cq, v at cq + ck
  long long ld;
  const float* bias;           // [cq + ck + cv] or null
  const float* taps_w;         // [taps, cq + ck + cv] (tap `taps - 1` on the token itself), or null with taps == 1: as it is
  float* history;              // [slots, taps - 1, cq + ck + cv] (null with taps == 1)
  const int *positions, *seq_of_token, *slots, *len_after, *seq_starts;
  int taps;
  int H, G, d, dv;             // query heads, key/value heads, size of a map's queries and keys, of the values
  int pk, pv;                  // elements between packed heads (and of a cache row): >= d, >= dv; zeros behind a head's own
  float temp_coef;
  int temp_every;              // 0: no temperature
  const int* page_table;
  int max_pages, ring_rows;
};

// u(position p of token t's sequence, channel c): the projected value with its bias, from the step's rows where the
// step holds p, else from the history (zero before the sequence's start).
__device__ __forceinline__ float conv_input(const AfConvArgs& a, int t, int pos, int p, int first_row, int first_pos,
                                            int slot, int C, int c) {
  if (p < 0) return 0.f;
  if (p >= first_pos) {
    const float v = a.proj[(size_t)(t - (pos - p)) * a.ld + c];
    return a.bias != nullptr ? v + a.bias[c] : v;
  }
  const int k = first_pos - p;                                   // 1 .. taps - 1 positions before the step
  return a.history[((size_t)slot * (a.taps - 1) + (a.taps - 1 - k)) * C + c];
}

// VEC packed elements a thread (neighbours within one head; VEC divides every head's sizes and pitches): block (x, y)
// takes elements 256 VEC y .. of token x's packed row (the q heads, then the k heads, then the v heads, padding
// included).  Where an element comes from and where it goes is worked out once for the VEC of them.
template <typename T, int VEC>
__global__ void __launch_bounds__(256)
conv_pack_kernel(T* __restrict__ qkv, long long out_stride, AfConvArgs a, T* __restrict__ kcache, T* __restrict__ vcache) {
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int cq = a.H * 2 * a.d, ck = a.G * 2 * a.d, cv = a.G * a.dv, C = cq + ck + cv;
  const int rep = a.H / a.G;
  const int nq = 2 * a.H, nk = 2 * a.G;
  const int n_q = nq * a.pk, n_k = nk * a.pk, n_v = nk * a.pv;
  const int i = (blockIdx.y * 256 + threadIdx.x) * VEC;
  if (i >= n_q + n_k + n_v) return;
  // the channel of the projection that the first element is made from (-1: padding), and where it goes in a cache row
  int c = -1, head = 0, e = 0, kind = 0;            // kind 0: q, 1: k, 2: v
  if (i < n_q) {
    head = i / a.pk, e = i - head * a.pk;
    const int g = head / (2 * rep), m = (head / rep) & 1, j = head % rep;
    if (e < a.d) c = ((g * rep + j) * 2 + m) * a.d + e;
  } else if (i < n_q + n_k) {
    const int x = i - n_q;
    head = x / a.pk, e = x - head * a.pk, kind = 1;
    if (e < a.d) c = cq + head * a.d + e;           // (head = 2 g + m, as the projection lays them out)
  } else {
    const int x = i - n_q - n_k;
    head = x / a.pv, e = x - head * a.pv, kind = 2;
    if (e < a.dv) c = cq + ck + (head >> 1) * a.dv + e;
  }
  const int taps = a.taps;
  float w[8][VEC], bias[VEC];
#pragma unroll
  for (int x = 0; x < VEC; ++x) bias[x] = (c >= 0 && a.bias != nullptr) ? a.bias[c + x] : 0.f;
  if (c >= 0 && a.taps_w != nullptr) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int x = 0; x < VEC; ++x) w[j][x] = j < taps ? a.taps_w[(size_t)j * C + c + x] : 0.f;
  }
  const int pos = a.positions[t];
  const int seq = a.seq_of_token[t];
  const int slot = a.slots[seq];
  const int first_pos = pos - (t - a.seq_starts[seq]);
  T* cache = nullptr;
  if (kind != 0 && kcache != nullptr && slot >= 0 && !(a.ring_rows > 0 && pos + a.ring_rows < a.len_after[seq])) {
    const int r = a.ring_rows > 0 ? pos % a.ring_rows : pos;
    if (AF_INDEX_OK(pos >= 0 && r / AF_PAGE < a.max_pages, r)) {
      const int page = a.page_table[(size_t)slot * a.max_pages + r / AF_PAGE];
      if (AF_INDEX_OK(page >= 0, page)) {
        const size_t at = ((size_t)page * nk + head) * AF_PAGE + r % AF_PAGE;
        cache = kind == 1 ? kcache + at * a.pk + e : vcache + at * a.pv + e;
      }
    }
  }
  pdl_wait();
  a.proj = pdl_fresh(a.proj);
  float v[VEC];
#pragma unroll
  for (int x = 0; x < VEC; ++x) v[x] = 0.f;
  if (c >= 0) {
    if (a.taps_w == nullptr) {
#pragma unroll
      for (int x = 0; x < VEC; ++x) v[x] = a.proj[(size_t)t * a.ld + c + x] + bias[x];
    } else {
      // the inputs of all taps first (they do not depend on one another), then the sums in tap order
      float u[8][VEC];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int x = 0; x < VEC; ++x) u[j][x] = 0.f;
        if (j >= taps) continue;
        const int p = pos - (taps - 1) + j;
        if (p < 0) continue;
        if (p >= first_pos) {
          const float* src = a.proj + (size_t)(t - (pos - p)) * a.ld + c;
#pragma unroll
          for (int x = 0; x < VEC; ++x) u[j][x] = src[x] + bias[x];
        } else if (slot >= 0) {
          const float* src = a.history + ((size_t)slot * (taps - 1) + (taps - 1 - (first_pos - p))) * C + c;
#pragma unroll
          for (int x = 0; x < VEC; ++x) u[j][x] = src[x];
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < taps) {
#pragma unroll
          for (int x = 0; x < VEC; ++x) v[x] = fmaf(w[j][x], u[j][x], v[x]);
        }
    }
    if (kind == 0 && a.temp_every > 0) {
      const float temp = 1.f + a.temp_coef * logf((float)((pos + 1) / a.temp_every + 1));
#pragma unroll
      for (int x = 0; x < VEC; ++x) v[x] *= temp;
    }
  }
  T* dst = qkv + (size_t)t * out_stride + i;
#pragma unroll
  for (int x = 0; x < VEC; ++x) {
    const T out = from_f32<T>(v[x]);
    dst[x] = out;
    if (cache != nullptr) cache[x] = out;
  }
}

// The same for more than eight taps: a loop over the taps, nothing held in registers.
template <typename T>
__global__ void __launch_bounds__(256)
conv_pack_long_kernel(T* __restrict__ qkv, long long out_stride, AfConvArgs a, T* __restrict__ kcache,
                      T* __restrict__ vcache) {
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int cq = a.H * 2 * a.d, ck = a.G * 2 * a.d, cv = a.G * a.dv, C = cq + ck + cv;
  const int rep = a.H / a.G;
  const int nq = 2 * a.H, nk = 2 * a.G;
  const int n_q = nq * a.pk, n_k = nk * a.pk, n_v = nk * a.pv;
  const int i = blockIdx.y * 256 + threadIdx.x;
  if (i >= n_q + n_k + n_v) return;
  int c = -1, head = 0, e = 0, kind = 0;
  if (i < n_q) {
    head = i / a.pk, e = i - head * a.pk;
    const int g = head / (2 * rep), m = (head / rep) & 1, j = head % rep;
    if (e < a.d) c = ((g * rep + j) * 2 + m) * a.d + e;
  } else if (i < n_q + n_k) {
    const int x = i - n_q;
    head = x / a.pk, e = x - head * a.pk, kind = 1;
    if (e < a.d) c = cq + head * a.d + e;
  } else {
    const int x = i - n_q - n_k;
    head = x / a.pv, e = x - head * a.pv, kind = 2;
    if (e < a.dv) c = cq + ck + (head >> 1) * a.dv + e;
  }
  const int pos = a.positions[t];
  const int seq = a.seq_of_token[t];
  const int slot = a.slots[seq];
  const int first_row = a.seq_starts[seq];
  const int first_pos = pos - (t - first_row);
  T* cache = nullptr;
  if (kind != 0 && kcache != nullptr && slot >= 0 && !(a.ring_rows > 0 && pos + a.ring_rows < a.len_after[seq])) {
    const int r = a.ring_rows > 0 ? pos % a.ring_rows : pos;
    if (AF_INDEX_OK(pos >= 0 && r / AF_PAGE < a.max_pages, r)) {
      const int page = a.page_table[(size_t)slot * a.max_pages + r / AF_PAGE];
      if (AF_INDEX_OK(page >= 0, page)) {
        const size_t at = ((size_t)page * nk + head) * AF_PAGE + r % AF_PAGE;
        cache = kind == 1 ? kcache + at * a.pk + e : vcache + at * a.pv + e;
      }
    }
  }
  pdl_wait();
  a.proj = pdl_fresh(a.proj);
  float v = 0.f;
  if (c >= 0) {
    for (int j = 0; j < a.taps; ++j) {
      const int p = pos - (a.taps - 1) + j;
      if (p < 0 || (p < first_pos && slot < 0)) continue;
      v = fmaf(a.taps_w[(size_t)j * C + c], conv_input(a, t, pos, p, first_row, first_pos, slot, C, c), v);
    }
    if (kind == 0 && a.temp_every > 0) v *= 1.f + a.temp_coef * logf((float)((pos + 1) / a.temp_every + 1));
  }
  const T out = from_f32<T>(v);
  qkv[(size_t)t * out_stride + i] = out;
  if (cache != nullptr) *cache = out;
}

// One thread a (sequence, channel): the history after the step = the last taps - 1 of (history, the step's values).
__global__ void __launch_bounds__(256)
conv_history_kernel(AfConvArgs a, int C) {
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int slot = a.slots[seq];
  if (c >= C || slot < 0) return;
  const int first = a.seq_starts[seq], n = a.seq_starts[seq + 1] - first;
  const int keep = a.taps - 1;
  float* h = a.history + (size_t)slot * keep * C + c;
  const float b = a.bias != nullptr ? a.bias[c] : 0.f;
  if (n >= keep) {
    for (int i = 0; i < keep; ++i) h[(size_t)i * C] = a.proj[(size_t)(first + n - keep + i) * a.ld + c] + b;
    return;
  }
  for (int i = 0; i < keep - n; ++i) h[(size_t)i * C] = h[(size_t)(i + n) * C];      // (ascending: a value is read before its place is written)
  for (int i = keep - n; i < keep; ++i) h[(size_t)i * C] = a.proj[(size_t)(first + n - keep + i) * a.ld + c] + b;
}

AF_EXPORT int af_conv_pack(void* qkv, int dtype, long long out_stride, const float* proj, long long ld, const float* bias,
                           const float* taps_w, float* history, const int* positions, const int* seq_of_token,
                           const int* slots, const int* len_after, const int* seq_starts, int n_tokens, int n_seqs, int taps,
                           int H, int G, int d, int dv, int pk, int pv, float temp_coef, int temp_every, void* kcache,
                           void* vcache, const int* page_table, int max_pages, int ring_rows, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && H > 0 && G > 0 && H % G == 0 && d > 0 && dv > 0 && pk >= d && pv >= dv && taps >= 1,
             "af_conv_pack: bad sizes");
  AF_REQUIRE(taps == 1 || (taps_w != nullptr && history != nullptr), "af_conv_pack: a convolution needs its taps and a history");
  AF_REQUIRE(ring_rows % AF_PAGE == 0, "af_conv_pack: ring rows %d not whole pages", ring_rows);
  AF_REQUIRE((kcache == nullptr) == (vcache == nullptr), "af_conv_pack: key and value pages, or neither");
  AfConvArgs a{proj, ld, bias, taps_w, history, positions, seq_of_token, slots, len_after, seq_starts, taps, H, G, d, dv,
               pk, pv, temp_coef, temp_every, page_table, max_pages, ring_rows};
  const int n_el = (2 * H + 2 * G) * pk + 2 * G * pv;
  const dim3 grid(n_tokens, (n_el + 255) / 256);
  AF_REQUIRE(grid.y < 65536, "af_conv_pack: rows of %d elements are too long for one grid", n_el);
  if (taps <= 8 && d % 4 == 0 && dv % 4 == 0 && pk % 4 == 0 && pv % 4 == 0) {
    const dim3 grid4(n_tokens, (n_el / 4 + 255) / 256);
    AF_DISPATCH_DTYPE(dtype, T, af_launch(conv_pack_kernel<T, 4>, grid4, dim3(256), 0, stream, (T*)qkv, out_stride, a,
                                          (T*)kcache, (T*)vcache));
  } else if (taps <= 8) {
    AF_DISPATCH_DTYPE(dtype, T, af_launch(conv_pack_kernel<T, 1>, grid, dim3(256), 0, stream, (T*)qkv, out_stride, a,
                                          (T*)kcache, (T*)vcache));
  } else {
    AF_DISPATCH_DTYPE(dtype, T, af_launch(conv_pack_long_kernel<T>, grid, dim3(256), 0, stream, (T*)qkv, out_stride, a,
                                          (T*)kcache, (T*)vcache));
  }
  AF_COUNT_LAUNCH("af_conv_pack");
  if (taps > 1) {
    const int C = H * 2 * d + G * 2 * d + G * dv;
    AF_REQUIRE(n_seqs > 0 && n_seqs < 65536, "af_conv_pack: too many sequences for one grid");
    af_launch(conv_history_kernel, dim3((C + 255) / 256, n_seqs), dim3(256), 0, stream, a, C);
    AF_COUNT_LAUNCH("af_conv_pack");
  }
  return 0;
}

// ctx [tokens, 2 H pv] (heads as conv_pack orders the queries) -> y [tokens, y_stride]: heads of dv values side by
// side, then `ones` columns of 1, then zeros up to y_stride.  gate: float32 rows [tokens, H dv] (null: no gate).
template <typename T>
__global__ void __launch_bounds__(256)
diff_join_kernel(T* __restrict__ y, long long y_stride, const T* __restrict__ ctx, long long ctx_stride,
                 const float* __restrict__ gate, long long gate_ts, int H, int G, int dv, int pv, float lambda, float eps,
                 float post, int ones) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int rep = H / G;
  const T* c = ctx + (size_t)t * ctx_stride;
  T* out = y + (size_t)t * y_stride;
  for (int h = warp; h < H; h += nwarp) {
    const int g = h / rep, j = h % rep;
    const T* a1 = c + (size_t)(g * 2 * rep + j) * pv;
    const T* a2 = c + (size_t)(g * 2 * rep + rep + j) * pv;
    float ss = 0.f;
    for (int e = lane; e < dv; e += 32) {
      const float o = to_f32<T>(a1[e]) - lambda * to_f32<T>(a2[e]);
      ss += o * o;
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)dv + eps) * post;
    for (int e = lane; e < dv; e += 32) {
      float o = (to_f32<T>(a1[e]) - lambda * to_f32<T>(a2[e])) * inv;
      if (gate != nullptr) o *= 1.f / (1.f + expf(-gate[(size_t)t * gate_ts + h * dv + e]));
      out[h * dv + e] = from_f32<T>(o);
    }
  }
  for (int i = H * dv + threadIdx.x; i < y_stride; i += blockDim.x) out[i] = from_f32<T>(i < H * dv + ones ? 1.f : 0.f);
}

AF_EXPORT int af_diff_join(void* y, long long y_stride, const void* ctx, long long ctx_stride, int dtype, const float* gate,
                           long long gate_ts, int n_tokens, int H, int G, int dv, int pv, float lambda, float eps, float post,
                           int ones, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && H > 0 && G > 0 && H % G == 0 && dv > 0 && pv >= dv && y_stride >= (long long)H * dv + ones,
             "af_diff_join: bad sizes");
  AF_DISPATCH_DTYPE(dtype, T, af_launch(diff_join_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, (T*)y, y_stride,
                                        (const T*)ctx, ctx_stride, gate, gate_ts, H, G, dv, pv, lambda, eps, post, ones));
  AF_CHECK_LAUNCH("af_diff_join");
}
