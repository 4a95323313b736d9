// Rotary position encoding with the cache write, and the plain attention
// kernels (one warp per query row and head, keys in order).  They serve the
// 32-bit path and stand beside the faster bfloat16 kernels as their twins.
//
// Cache of one layer: pages [n_pages][n_kv_heads][AF_PAGE][head_dim] for K and
// for V.  A sequence's page table maps row / AF_PAGE to a page.  A layer with
// a window keeps rows modulo `ring_rows` (a multiple of AF_PAGE, >= window).
#include "common.cuh"

#define AF_MAX_HD 640
#define AF_HD_SLICES (AF_MAX_HD / 32)

// ---------------------------------------------------------------- rope + cache write

// One block per (token, head) of the packed row [q heads | k heads | v heads].
// Rotates q and k heads in place (32-bit angles and arithmetic) and, when a
// cache is given, stores the rotated k and the v in the row's page.  The row
// may arrive as split-K partial sums (float), added in index order first.
template <typename T>
__device__ __forceinline__ float rope_src(const T* row, const float* parts, int n_parts, size_t part_stride,
                                          int i) {
  if (parts == nullptr) return to_f32(row[i]);
  // (16 loads in flight: a product of up to 16 splits costs one round trip; the sums go on in index order)
  float acc[16];
  float v = 0.f;
  for (int p0 = 0; p0 < n_parts; p0 += 16) {
#pragma unroll
    for (int u = 0; u < 16; ++u) acc[u] = p0 + u < n_parts ? parts[(size_t)(p0 + u) * part_stride + i] : 0.f;
#pragma unroll
    for (int u = 0; u < 16; ++u) v += acc[u];
  }
  return v;
}

template <typename T>
__global__ void rope_cache_kernel(T* __restrict__ qkv, int row_stride, const float* __restrict__ parts,
                                  int n_parts, size_t part_stride, const int* __restrict__ positions,
                                  const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                                  const int* __restrict__ len_after, const float* __restrict__ inv_freq,
                                  int nq, int nkv, int hd, int rot_dim, int pairing,
                                  T* __restrict__ kcache, T* __restrict__ vcache,
                                  const int* __restrict__ page_table, int max_pages, int ring_rows) {
  pdl_launch_dependents();
  // Positions, slots, lengths, the page table and the frequencies are inputs of the step, not
  // results of the kernel before: the row's place in the cache and the first pair's sine and
  // cosine are worked out before the wait for that kernel.
  const int t = blockIdx.x, head = blockIdx.y;
  const int pos = positions[t];
  T* row = qkv + (size_t)t * row_stride + (size_t)head * hd;
  const float* pr = parts ? parts + (size_t)t * (nq + 2 * nkv) * hd + (size_t)head * hd : nullptr;  // (read after the wait)
  const int half = rot_dim / 2;
  // where this head's row goes in the cache (k and v heads only)
  T* dst = nullptr;
  if (kcache != nullptr && head >= nq) {
    const int seq = seq_of_token[t];
    const int slot = slots[seq];
    // of the tokens of this step that share a ring row only the last is kept; padding rows are skipped
    if (slot >= 0 && !(ring_rows > 0 && pos + ring_rows < len_after[seq])) {
      const int r = ring_rows > 0 ? pos % ring_rows : pos;
      if (AF_INDEX_OK(pos >= 0 && r / AF_PAGE < max_pages, r)) {
        const int page = page_table[(size_t)slot * max_pages + r / AF_PAGE];
        const bool is_v = head >= nq + nkv;
        const int h = head - nq - (is_v ? nkv : 0);
        if (AF_INDEX_OK(page >= 0, page))
          dst = (is_v ? vcache : kcache) + (((size_t)page * nkv + h) * AF_PAGE + r % AF_PAGE) * hd;
      }
    }
  }
  const bool rotate = head < nq + nkv;
  float s0 = 0.f, c0 = 1.f;
  if (rotate && threadIdx.x < half) sincosf((float)pos * inv_freq[threadIdx.x], &s0, &c0);
  pdl_wait();
  pr = pdl_fresh(pr);
  row = pdl_fresh(row);
  // rotary pairs
  for (int p = threadIdx.x; p < half; p += blockDim.x) {
    const int i0 = pairing == AF_PAIR_HALF ? p : 2 * p;
    const int i1 = pairing == AF_PAIR_HALF ? p + half : 2 * p + 1;
    float a = rope_src(row, pr, n_parts, part_stride, i0);
    float b = rope_src(row, pr, n_parts, part_stride, i1);
    if (rotate) {
      float s = s0, c = c0;
      if (p != threadIdx.x) sincosf((float)pos * inv_freq[p], &s, &c);
      const float ra = a * c - b * s, rb = b * c + a * s;
      a = ra;
      b = rb;
    }
    const T ta = from_f32<T>(a), tb = from_f32<T>(b);
    if (rotate || pr != nullptr) {
      row[i0] = ta;
      row[i1] = tb;
    }
    if (dst != nullptr) {
      dst[i0] = ta;
      dst[i1] = tb;
    }
  }
  // elements beyond the rotary part
  for (int i = rot_dim + threadIdx.x; i < hd; i += blockDim.x) {
    const T v = from_f32<T>(rope_src(row, pr, n_parts, part_stride, i));
    if (pr != nullptr) row[i] = v;
    if (dst != nullptr) dst[i] = v;
  }
}

// The same for bfloat16 rows without partial sums, half-split pairs over the
// whole head and head_dim % 16 == 0: one block per token, 16-byte loads and
// stores, eight pairs a thread.
__global__ void __launch_bounds__(256)
rope_cache_vec_kernel(__nv_bfloat16* __restrict__ qkv, long long row_stride, const int* __restrict__ positions,
                      const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                      const int* __restrict__ len_after, const float* __restrict__ inv_freq,
                      const float2* __restrict__ table, int nq, int nkv, int hd,
                      __nv_bfloat16* __restrict__ kcache, __nv_bfloat16* __restrict__ vcache,
                      const int* __restrict__ page_table, int max_pages, int ring_rows) {
  pdl_launch_dependents();
  // (positions, slots, lengths, page table and frequencies are inputs of the step: the row's place in
  // the cache and the sines and cosines are worked out before the wait for the kernel in front)
  const int t = blockIdx.x;
  const int pos = positions[t];
  __nv_bfloat16* row = qkv + (size_t)t * row_stride;
  const int half = hd / 2;
  const int per_head = half / 8;                 // 16-byte pieces of a half head
  const int n_heads = nq + 2 * nkv;
  // where this token's k and v rows go in the cache
  size_t dst_row = 0;
  bool store = false;
  if (kcache != nullptr) {
    const int seq = seq_of_token[t];
    const int slot = slots[seq];
    if (slot >= 0 && !(ring_rows > 0 && pos + ring_rows < len_after[seq])) {
      const int r = ring_rows > 0 ? pos % ring_rows : pos;
      if (AF_INDEX_OK(pos >= 0 && r / AF_PAGE < max_pages, r)) {
        const int page = page_table[(size_t)slot * max_pages + r / AF_PAGE];
        dst_row = ((size_t)page * nkv) * AF_PAGE + r % AF_PAGE;   // + h * AF_PAGE rows for kv head h
        store = AF_INDEX_OK(page >= 0, page);
      }
    }
  }
  // a thread's pieces all have the same place in their heads when the block's size is a multiple of
  // the pieces of a head (it is for head sizes up to 512 that divide so): its 8 pairs' angles are fixed
  const bool fixed_c = blockDim.x % per_head == 0;
  float sn0[8], cs0[8];
  if (fixed_c && table == nullptr) {
    const int c = threadIdx.x % per_head;
#pragma unroll
    for (int e = 0; e < 8; ++e) sincosf((float)pos * inv_freq[c * 8 + e], &sn0[e], &cs0[e]);
  }
  pdl_wait();
  row = pdl_fresh(row);
  if (fixed_c && table != nullptr) {
    // the step's table of (cos, sin), made once for all layers by the same arithmetic (a kernel of this step
    // wrote it: read after the wait)
    const float4* tp = reinterpret_cast<const float4*>(pdl_fresh(table) + (size_t)t * half + (threadIdx.x % per_head) * 8);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float4 v = tp[e];
      cs0[2 * e] = v.x, sn0[2 * e] = v.y, cs0[2 * e + 1] = v.z, sn0[2 * e + 1] = v.w;
    }
  }
  for (int i = threadIdx.x; i < n_heads * per_head; i += blockDim.x) {
    const int head = i / per_head, c = i - head * per_head;
    __nv_bfloat16* x = row + (size_t)head * hd + c * 8;
    uint4 lo = *reinterpret_cast<const uint4*>(x);
    uint4 hi = *reinterpret_cast<const uint4*>(x + half);
    if (head < nq + nkv) {
      uint32_t* lw = reinterpret_cast<uint32_t*>(&lo);
      uint32_t* hw = reinterpret_cast<uint32_t*>(&hi);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float a[2] = {__uint_as_float(lw[j] << 16), __uint_as_float(lw[j] & 0xffff0000u)};
        float b[2] = {__uint_as_float(hw[j] << 16), __uint_as_float(hw[j] & 0xffff0000u)};
        float ra[2], rb[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          float sn = sn0[2 * j + e], cs = cs0[2 * j + e];
          if (!fixed_c) sincosf((float)pos * inv_freq[c * 8 + 2 * j + e], &sn, &cs);
          ra[e] = a[e] * cs - b[e] * sn;
          rb[e] = b[e] * cs + a[e] * sn;
        }
        __nv_bfloat162 pa = __floats2bfloat162_rn(ra[0], ra[1]), pb = __floats2bfloat162_rn(rb[0], rb[1]);
        lw[j] = *reinterpret_cast<uint32_t*>(&pa);
        hw[j] = *reinterpret_cast<uint32_t*>(&pb);
      }
      *reinterpret_cast<uint4*>(x) = lo;
      *reinterpret_cast<uint4*>(x + half) = hi;
    }
    if (store && head >= nq) {
      const bool is_v = head >= nq + nkv;
      const int h = head - nq - (is_v ? nkv : 0);
      __nv_bfloat16* d = (is_v ? vcache : kcache) + (dst_row + (size_t)h * AF_PAGE) * hd + c * 8;
      *reinterpret_cast<uint4*>(d) = lo;
      *reinterpret_cast<uint4*>(d + half) = hi;
    }
  }
}

// `parts` (optional): float [n_parts, n_tokens, row width] partial sums of the
// rows, part_stride elements apart; they are added in order into qkv first.
AF_EXPORT int af_rope_cache_write(void* qkv, int dtype, int row_stride, const float* parts, int n_parts,
                                  long long part_stride, const int* positions,
                                  const int* seq_of_token, const int* slots, const int* len_after,
                                  const float* inv_freq, const float* table, int n_tokens, int nq, int nkv, int hd,
                                  int rot_dim, int pairing, void* kcache, void* vcache,
                                  const int* page_table, int max_pages, int ring_rows,
                                  cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && nq > 0 && nkv > 0 && hd > 0, "af_rope_cache_write: bad sizes");
  AF_REQUIRE(rot_dim >= 0 && rot_dim <= hd && rot_dim % 2 == 0,
             "af_rope_cache_write: rotary dim %d must be even and <= head_dim %d", rot_dim, hd);
  AF_REQUIRE(pairing == AF_PAIR_HALF || pairing == AF_PAIR_ADJACENT, "af_rope_cache_write: pairing");
  AF_REQUIRE(ring_rows % AF_PAGE == 0, "af_rope_cache_write: ring rows %d not whole pages", ring_rows);
  AF_REQUIRE((kcache == nullptr) == (vcache == nullptr), "af_rope_cache_write: k and v cache");
  if (dtype == AF_BF16 && parts == nullptr && pairing == AF_PAIR_HALF && rot_dim == hd && hd % 16 == 0 &&
      row_stride % 8 == 0 && ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)kcache & 15) == 0 &&
      ((uintptr_t)vcache & 15) == 0 && n_tokens >= 64) {
    af_launch(rope_cache_vec_kernel, dim3(n_tokens), dim3(256), 0, stream, (__nv_bfloat16*)qkv, (long long)row_stride,
              positions, seq_of_token, slots, len_after, inv_freq,
              ((uintptr_t)table & 15) == 0 ? reinterpret_cast<const float2*>(table) : nullptr, nq, nkv, hd, (__nv_bfloat16*)kcache,
              (__nv_bfloat16*)vcache, page_table, max_pages, ring_rows);
    AF_CHECK_LAUNCH("af_rope_cache_write");
  }
  AF_DISPATCH_DTYPE(dtype, T,
                    af_launch(rope_cache_kernel<T>, dim3(dim3(n_tokens, nq + 2 * nkv)), dim3(hd / 2 < 32 ? 32 : (hd / 2 > 256 ? 256 : hd / 2)), 0, stream, 
                        (T*)qkv, row_stride, parts, n_parts, (size_t)part_stride, positions, seq_of_token,
                        slots, len_after, inv_freq, nq,
                        nkv, hd, rot_dim, pairing, (T*)kcache, (T*)vcache, page_table, max_pages,
                        ring_rows));
  AF_CHECK_LAUNCH("af_rope_cache_write");
}

// ---------------------------------------------------------------- tables of a step

// (cos, sin) of position * frequency for every token and rotary pair: float [n_tokens][half][2].  Made once
// per step for all layers that rotate by the same frequencies; 32-bit angles as in the rotary kernels.
__global__ void rope_table_kernel(float2* __restrict__ table, const int* __restrict__ positions,
                                  const float* __restrict__ inv_freq, int half) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const float pos = (float)positions[t];
  for (int p = threadIdx.x; p < half; p += blockDim.x) {
    float s, c;
    sincosf(pos * inv_freq[p], &s, &c);
    table[(size_t)t * half + p] = make_float2(c, s);
  }
}

// The same from 64-bit frequencies, the angle and its reduction in 64 bits (a position of some thousands times a
// frequency near 1 loses the last bits of a 32-bit angle): for designs whose tolerance is that of 32-bit logits.
__global__ void rope_table_precise_kernel(float2* __restrict__ table, const int* __restrict__ positions,
                                          const double* __restrict__ inv_freq, int half) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const double pos = (double)positions[t];
  for (int p = threadIdx.x; p < half; p += blockDim.x) {
    double s, c;
    sincos(pos * inv_freq[p], &s, &c);
    table[(size_t)t * half + p] = make_float2((float)c, (float)s);
  }
}

AF_EXPORT int af_rope_table_precise(float* table, const int* positions, const double* inv_freq, int n_tokens, int half,
                                    cudaStream_t stream) {
  if (n_tokens == 0 || half == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && half > 0 && ((uintptr_t)table & 7) == 0, "af_rope_table_precise: bad sizes");
  af_launch(rope_table_precise_kernel, dim3(n_tokens), dim3(half < 32 ? 32 : (half > 256 ? 256 : half)), 0, stream,
            reinterpret_cast<float2*>(table), positions, inv_freq, half);
  AF_CHECK_LAUNCH("af_rope_table_precise");
}

AF_EXPORT int af_rope_table(float* table, const int* positions, const float* inv_freq, int n_tokens, int half,
                            cudaStream_t stream) {
  if (n_tokens == 0 || half == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && half > 0 && ((uintptr_t)table & 7) == 0, "af_rope_table: bad sizes");
  af_launch(rope_table_kernel, dim3(n_tokens), dim3(half < 32 ? 32 : (half > 256 ? 256 : half)), 0, stream,
            reinterpret_cast<float2*>(table), positions, inv_freq, half);
  AF_CHECK_LAUNCH("af_rope_table");
}

// Where each token's keys and values go in the cache of one group of layers: rows[t] = page * nkv * AF_PAGE +
// row in page (the row of kv head 0; head h lies h * AF_PAGE rows further), or -1 when the token is not stored
// (a padding row; a token of a long prompt whose ring row a later token of the same step takes).
__global__ void kv_rows_kernel(int* __restrict__ rows, const int* __restrict__ positions,
                               const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                               const int* __restrict__ len_after, const int* __restrict__ page_table, int max_pages,
                               int ring_rows, int nkv, int n_tokens) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_tokens) return;
  const int pos = positions[t], seq = seq_of_token[t], slot = slots[seq];
  int row = -1;
  if (slot >= 0 && !(ring_rows > 0 && pos + ring_rows < len_after[seq])) {
    const int r = ring_rows > 0 ? pos % ring_rows : pos;
    if (AF_INDEX_OK(pos >= 0 && r / AF_PAGE < max_pages, r)) {
      const int page = page_table[(size_t)slot * max_pages + r / AF_PAGE];
      if (AF_INDEX_OK(page >= 0, page)) row = page * nkv * AF_PAGE + r % AF_PAGE;
    }
  }
  rows[t] = row;
}

AF_EXPORT int af_kv_rows(int* rows, const int* positions, const int* seq_of_token, const int* slots,
                         const int* len_after, const int* page_table, int max_pages, int ring_rows, int nkv,
                         int n_tokens, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && nkv > 0 && ring_rows % AF_PAGE == 0, "af_kv_rows: bad sizes");
  af_launch(kv_rows_kernel, dim3((n_tokens + 127) / 128), dim3(128), 0, stream, rows, positions, seq_of_token, slots,
            len_after, page_table, max_pages, ring_rows, nkv, n_tokens);
  AF_CHECK_LAUNCH("af_kv_rows");
}

// ---------------------------------------------------------------- plain attention

// Online-softmax state of one (query, head) held by a warp: lane l owns the
// elements l, l + 32, ... of the head.  Keys have dk elements, values dv.
struct WarpAttn {
  float q[AF_HD_SLICES];
  float o[AF_HD_SLICES];
  float m, l;
};

// The first position that position `pos` sees.  AF_MASK_WINDOW: the last `size` positions, itself
// included; AF_MASK_CHUNK: its own chunk of `size` positions, chunks counted from position 0.  size <= 0: all.
__device__ __forceinline__ int first_visible(int pos, int size, int mask_kind) {
  if (size <= 0) return 0;
  return mask_kind == AF_MASK_CHUNK ? pos - pos % size : max(0, pos - size + 1);
}

// `sink` (or -inf): a term exp(sink) of the softmax's denominator that has no key and no value.
template <typename T>
__device__ __forceinline__ void attn_load_q(WarpAttn& st, const T* q, int dk, int lane, float sink = -INFINITY) {
#pragma unroll
  for (int e = 0; e < AF_HD_SLICES; ++e) {
    const int d = lane + 32 * e;
    st.q[e] = d < dk ? to_f32(q[d]) : 0.f;
    st.o[e] = 0.f;
  }
  st.m = sink;
  st.l = sink > -INFINITY ? 1.f : 0.f;
}

template <typename T>
__device__ __forceinline__ void attn_key(WarpAttn& st, const T* k, const T* v, int dk, int dv, int lane,
                                         float scale, float cap, float bias) {
  float dot = 0.f;
#pragma unroll
  for (int e = 0; e < AF_HD_SLICES; ++e) {
    const int d = lane + 32 * e;
    if (d < dk) dot += st.q[e] * to_f32(k[d]);
  }
  dot = warp_sum(dot);
  const float s = softcap_f32(dot * scale, cap) + bias;   // bias: a position encoding's slope * (key - query)
  const float m_new = fmaxf(st.m, s);
  const float corr = expf(st.m - m_new);  // exp(-inf) = 0 on the first key
  const float p = expf(s - m_new);
  st.l = st.l * corr + p;
#pragma unroll
  for (int e = 0; e < AF_HD_SLICES; ++e) {
    const int d = lane + 32 * e;
    if (d < dv) st.o[e] = st.o[e] * corr + p * to_f32(v[d]);
  }
  st.m = m_new;
}

// `factor`: what the head's output is multiplied by (an output gate; 1 without one).
template <typename T>
__device__ __forceinline__ void attn_store(const WarpAttn& st, T* out, int dv, int lane, float factor = 1.f) {
  const float inv = st.l > 0.f ? factor / st.l : 0.f;
#pragma unroll
  for (int e = 0; e < AF_HD_SLICES; ++e) {
    const int d = lane + 32 * e;
    if (d < dv) out[d] = from_f32<T>(st.o[e] * inv);
  }
}

__device__ __forceinline__ float gate_factor(const float* gate, long long gate_stride, int row, int h) {
  return gate ? 1.f / (1.f + expf(-gate[(size_t)row * gate_stride + h])) : 1.f;
}

// Prompts that start at position 0: keys and values are the step's own rows.
// Warp w of the grid handles (token, head) = (w / nq, w % nq).  `hd` is the key size, `dv` the value
// size; `sinks` (float [nq]) and `gate` (float logits, row t and column h at gate[t * gate_stride + h]:
// the head's output is multiplied by their sigmoid) may be null.
template <typename T>
__global__ void attn_prefill_plain_kernel(T* __restrict__ out, int out_stride, const T* __restrict__ q,
                                          int q_stride, const T* __restrict__ k, int k_stride,
                                          const T* __restrict__ v, int v_stride,
                                          const int* __restrict__ positions,
                                          int n_tokens, int nq, int nkv, int hd, int dv, float scale, float cap,
                                          int window, int mask_kind, const float* __restrict__ slopes,
                                          const float* __restrict__ sinks, const float* __restrict__ gate,
                                          long long gate_stride) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)n_tokens * nq) return;
  const int t = (int)(w / nq), h = (int)(w % nq);
  const int g = h / (nq / nkv);
  const int pos = positions[t];          // position inside its sequence
  const int first_row = t - pos;         // row of the sequence's position 0
  WarpAttn st;
  attn_load_q(st, q + (size_t)t * q_stride + (size_t)h * hd, hd, lane, sinks ? sinks[h] : -INFINITY);
  const int lo = first_visible(pos, window, mask_kind);
  const float slope = slopes ? slopes[h] : 0.f;
  for (int j = lo; j <= pos; ++j) {
    const size_t r = (size_t)(first_row + j);
    attn_key(st, k + r * k_stride + (size_t)g * hd, v + r * v_stride + (size_t)g * dv, hd, dv, lane, scale,
             cap, slope * (float)(j - pos));
  }
  attn_store(st, out + (size_t)t * out_stride + (size_t)h * dv, dv, lane, gate_factor(gate, gate_stride, t, h));
}

AF_EXPORT int af_attn_prefill_plain(void* out, int out_stride, const void* q, int q_stride,
                                    const void* k, int k_stride, const void* v, int v_stride, int dtype,
                                    const int* positions, int n_tokens, int nq, int nkv, int hd, int dv,
                                    float scale, float cap, int window, int mask_kind, const float* slopes,
                                    const float* sinks, const float* gate, long long gate_stride,
                                    cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  AF_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "af_attn_prefill_plain: heads %d, groups %d", nq, nkv);
  AF_REQUIRE(hd > 0 && hd <= AF_MAX_HD && dv > 0 && dv <= AF_MAX_HD,
             "af_attn_prefill_plain: key size %d or value size %d beyond %d", hd, dv, AF_MAX_HD);
  AF_REQUIRE(mask_kind == AF_MASK_WINDOW || mask_kind == AF_MASK_CHUNK, "af_attn_prefill_plain: mask kind %d", mask_kind);
  const long long warps = (long long)n_tokens * nq;
  const int wpb = 4;
  const long long blocks = (warps + wpb - 1) / wpb;
  AF_REQUIRE(blocks < (1ll << 31), "af_attn_prefill_plain: too many rows");
  AF_DISPATCH_DTYPE(dtype, T,
                    af_launch(attn_prefill_plain_kernel<T>, dim3((unsigned)blocks), dim3(wpb * 32), 0, stream, 
                        (T*)out, out_stride, (const T*)q, q_stride, (const T*)k, k_stride, (const T*)v,
                        v_stride, positions, n_tokens, nq, nkv, hd, dv, scale, cap, window, mask_kind, slopes,
                        sinks, gate, gate_stride));
  AF_CHECK_LAUNCH("af_attn_prefill_plain");
}

// One new token per sequence: keys and values come from the cache pages.
// `lens[b]` counts the new token, which the cache holds already.  Key pages hold rows of `hd` elements,
// value pages rows of `dv`; with no value pages (vcache null) a value is the first `dv` elements of its key row.
// A warp per (sequence, head, split): with n_splits > 1 the visible keys are cut into that many equal runs and
// a warp leaves its run's unnormalised output, maximum and sum in part_o / part_ml for the merge kernel.
template <typename T>
__global__ void attn_decode_plain_kernel(T* __restrict__ out, int out_stride, const T* __restrict__ q,
                                         int q_stride, const T* __restrict__ kcache,
                                         const T* __restrict__ vcache, const int* __restrict__ page_table,
                                         int max_pages, const int* __restrict__ slots,
                                         const int* __restrict__ lens, int batch, int nq, int nkv, int hd, int dv,
                                         float scale, float cap, int window, int mask_kind, int ring_rows,
                                         const float* __restrict__ slopes, const float* __restrict__ sinks,
                                         const float* __restrict__ gate, long long gate_stride, int n_splits,
                                         float* __restrict__ part_o, float* __restrict__ part_ml) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)batch * nq * n_splits) return;
  const int split = (int)(w % n_splits);
  const long long unit = w / n_splits;              // (sequence, head)
  const int b = (int)(unit / nq), h = (int)(unit % nq);
  const int g = h / (nq / nkv);
  const int slot = slots[b];
  T* o = out + (size_t)b * out_stride + (size_t)h * dv;
  if (slot < 0) {  // padding row
    if (split == 0)
      for (int d = lane; d < dv; d += 32) o[d] = from_f32<T>(0.f);
    if (n_splits > 1 && lane == 0) part_ml[2 * w] = -INFINITY, part_ml[2 * w + 1] = 0.f;
    return;
  }
  const int len = lens[b];
  const int pos = len - 1;
  WarpAttn st;
  // (with splits the sink joins in the merge)
  attn_load_q(st, q + (size_t)b * q_stride + (size_t)h * hd, hd, lane, sinks && n_splits == 1 ? sinks[h] : -INFINITY);
  int lo = first_visible(pos, window, mask_kind), hi = pos;
  if (n_splits > 1) {
    const int per = (pos - lo + n_splits) / n_splits;       // ceil((pos - lo + 1) / n_splits)
    lo += split * per;
    hi = min(pos, lo + per - 1);
  }
  const int* pt = page_table + (size_t)slot * max_pages;
  const float slope = slopes ? slopes[h] : 0.f;
  for (int j = lo; j <= hi; ++j) {
    const int r = ring_rows > 0 ? j % ring_rows : j;
    if (!AF_INDEX_OK(r / AF_PAGE < max_pages && pt[r / AF_PAGE] >= 0, r)) continue;
    const size_t row = ((size_t)pt[r / AF_PAGE] * nkv + g) * AF_PAGE + r % AF_PAGE;
    const T* kr = kcache + row * hd;
    attn_key(st, kr, vcache ? vcache + row * dv : kr, hd, dv, lane, scale, cap, slope * (float)(j - pos));
  }
  if (n_splits == 1) {
    attn_store(st, o, dv, lane, gate_factor(gate, gate_stride, b, h));
    return;
  }
  float* po = part_o + (size_t)w * dv;
#pragma unroll
  for (int e = 0; e < AF_HD_SLICES; ++e) {
    const int d = lane + 32 * e;
    if (d < dv) po[d] = st.o[e];
  }
  if (lane == 0) part_ml[2 * w] = st.m, part_ml[2 * w + 1] = st.l;
}

// Joins the splits of a (sequence, head): out = sum_s o_s e^(m_s - M) / (sum_s l_s e^(m_s - M) + e^(sink - M)),
// times the gate's factor.  One block per (sequence, head), threads over the value's elements.
template <typename T>
__global__ void __launch_bounds__(128)
attn_decode_plain_merge_kernel(T* __restrict__ out, int out_stride, const float* __restrict__ part_o,
                               const float* __restrict__ part_ml, const int* __restrict__ slots, int nq, int dv,
                               int n_splits, const float* __restrict__ sinks, const float* __restrict__ gate,
                               long long gate_stride) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, h = blockIdx.y;
  if (slots[b] < 0) return;                                  // (a padding row: the split kernel wrote zeros)
  const size_t u = ((size_t)b * nq + h) * n_splits;
  // every run's factor e^(m_s - M) / L once, in shared memory (up to 256 runs; more: worked out again by every thread)
  __shared__ float f_s[256];
  __shared__ float inv_s;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float M = sinks ? sinks[h] : -INFINITY;
    for (int s = lane; s < n_splits; s += 32) M = fmaxf(M, part_ml[2 * (u + s)]);
    M = warp_max(M);
    float L = 0.f;
    for (int s = lane; s < n_splits; s += 32) {
      const float m = part_ml[2 * (u + s)];
      const float f = m > -INFINITY ? expf(m - M) : 0.f;
      if (s < 256) f_s[s] = f;
      L += part_ml[2 * (u + s) + 1] * f;
    }
    L = warp_sum(L);
    if (sinks) L += expf(sinks[h] - M);
    if (lane == 0) inv_s = L > 0.f ? gate_factor(gate, gate_stride, b, h) / L : 0.f;
    if (n_splits > 256 && lane == 0) f_s[0] = M;       // (kept for the long way below)
  }
  __syncthreads();
  const float inv = inv_s;
  T* o = out + (size_t)b * out_stride + (size_t)h * dv;
  for (int d = threadIdx.x; d < dv; d += blockDim.x) {
    float acc = 0.f;
    if (n_splits <= 256) {
#pragma unroll 4
      for (int s = 0; s < n_splits; ++s) acc += part_o[(u + s) * dv + d] * f_s[s];
    } else {
      const float M = f_s[0];
      for (int s = 0; s < n_splits; ++s) {
        const float m = part_ml[2 * (u + s)];
        if (m > -INFINITY) acc += part_o[(u + s) * dv + d] * expf(m - M);
      }
    }
    o[d] = from_f32<T>(acc * inv);
  }
}

// `scratch`: n_splits > 1 needs batch * nq * n_splits * (dv + 2) floats.
AF_EXPORT int af_attn_decode_plain(void* out, int out_stride, const void* q, int q_stride,
                                   const void* kcache, const void* vcache, int dtype,
                                   const int* page_table, int max_pages, const int* slots,
                                   const int* lens, int batch, int nq, int nkv, int hd, int dv, float scale,
                                   float cap, int window, int mask_kind, int ring_rows, const float* slopes,
                                   const float* sinks, const float* gate, long long gate_stride, int n_splits,
                                   float* scratch, cudaStream_t stream) {
  if (batch == 0) return 0;
  AF_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "af_attn_decode_plain: heads %d, groups %d", nq, nkv);
  AF_REQUIRE(hd > 0 && hd <= AF_MAX_HD && dv > 0 && dv <= AF_MAX_HD && (vcache != nullptr || dv <= hd),
             "af_attn_decode_plain: key size %d or value size %d beyond %d (or values longer than the keys they lie in)",
             hd, dv, AF_MAX_HD);
  AF_REQUIRE(mask_kind == AF_MASK_WINDOW || mask_kind == AF_MASK_CHUNK, "af_attn_decode_plain: mask kind %d", mask_kind);
  AF_REQUIRE(ring_rows % AF_PAGE == 0 && (ring_rows == 0 || window > 0) && (window <= ring_rows || ring_rows == 0),
             "af_attn_decode_plain: window %d, ring rows %d", window, ring_rows);
  AF_REQUIRE(n_splits >= 1 && (n_splits == 1 || scratch != nullptr) && batch < 65536 && nq < 65536,
             "af_attn_decode_plain: %d splits need scratch memory", n_splits);
  const long long warps = (long long)batch * nq * n_splits;
  const int wpb = 4;
  const long long blocks = (warps + wpb - 1) / wpb;
  AF_REQUIRE(blocks < (1ll << 31), "af_attn_decode_plain: too many rows");
  float* part_o = scratch;
  float* part_ml = scratch ? scratch + (size_t)warps * dv : nullptr;
  AF_DISPATCH_DTYPE(dtype, T,
                    af_launch(attn_decode_plain_kernel<T>, dim3((unsigned)blocks), dim3(wpb * 32), 0, stream, 
                        (T*)out, out_stride, (const T*)q, q_stride, (const T*)kcache, (const T*)vcache,
                        page_table, max_pages, slots, lens, batch, nq, nkv, hd, dv, scale, cap, window, mask_kind,
                        ring_rows, slopes, sinks, gate, gate_stride, n_splits, part_o, part_ml));
  if (n_splits == 1) AF_CHECK_LAUNCH("af_attn_decode_plain");
  AF_COUNT_LAUNCH("af_attn_decode_plain");
  AF_DISPATCH_DTYPE(dtype, T,
                    af_launch(attn_decode_plain_merge_kernel<T>, dim3(batch, nq), dim3(128), 0, stream, (T*)out,
                              out_stride, (const float*)part_o, (const float*)part_ml, slots, nq, dv, n_splits, sinks,
                              gate, gate_stride));
  AF_CHECK_LAUNCH("af_attn_decode_plain");
}

// The merge alone, for kernels that leave runs in the same form (attention_latent.cu).
AF_EXPORT int af_attn_decode_merge_runs(void* out, int out_stride, int dtype, const float* part_o, const float* part_ml,
                                        const int* slots, int batch, int nq, int dv, int n_splits, const float* sinks,
                                        const float* gate, long long gate_stride, cudaStream_t stream) {
  if (batch == 0) return 0;
  AF_REQUIRE(batch > 0 && batch < 65536 && nq > 0 && nq < 65536 && dv > 0 && n_splits >= 1 && part_o && part_ml,
             "af_attn_decode_merge_runs: bad sizes");
  AF_DISPATCH_DTYPE(dtype, T,
                    af_launch(attn_decode_plain_merge_kernel<T>, dim3(batch, nq), dim3(128), 0, stream, (T*)out,
                              out_stride, part_o, part_ml, slots, nq, dv, n_splits, sinks, gate, gate_stride));
  AF_CHECK_LAUNCH("af_attn_decode_merge_runs");
}

// An output gate behind an attention kernel that has none of its own: x[t, h, :] *= sigmoid(gate[t, h]).
template <typename T>
__global__ void __launch_bounds__(256)
head_gate_kernel(T* __restrict__ x, long long x_stride, const float* __restrict__ gate, long long gate_stride,
                 int nq, int dv, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t at = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (at >= total) return;
  const int per_row = nq * dv;
  const size_t t = at / per_row;
  const int i = (int)(at - t * per_row);
  T* p = x + t * x_stride + i;
  *p = from_f32<T>(to_f32(*p) * gate_factor(gate, gate_stride, (int)t, i / dv));
}

AF_EXPORT int af_head_gate(void* x, long long x_stride, int dtype, const float* gate, long long gate_stride, int n_rows,
                           int nq, int dv, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  AF_REQUIRE(n_rows > 0 && nq > 0 && dv > 0 && gate != nullptr, "af_head_gate: bad sizes");
  const size_t total = (size_t)n_rows * nq * dv;
  const size_t blocks = (total + 255) / 256;
  AF_REQUIRE(blocks < (1ull << 31), "af_head_gate: too many rows");
  AF_DISPATCH_DTYPE(dtype, T,
                    af_launch(head_gate_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, (T*)x, x_stride, gate,
                              gate_stride, nq, dv, total));
  AF_CHECK_LAUNCH("af_head_gate");
}

// ---------------------------------------------------------------- norm + rope + cache write from a projection

// Queries and keys that are normalised per head, and values that may be the raw key projection.  The
// projection row of a token is float [q heads | k heads (| v heads of `dv` values)]; a warp per
// (token, q or k head):
//   x = the head's projection (+ its part of `bias`, float, laid out like the row)
//   n = x * rsqrt(mean(x^2) + eps) * weight   (weight of head_dim values shared by the heads; none: n = x)
//   r = the first rot_dim elements of n rotated by position * frequency (32-bit), cosines and sines
//       multiplied by `magnitude`; the rest kept
//   with `norm_after`: r / sqrt(mean(r^2) + eps) over the whole head (no weight)
// and written to the packed row [q | k | v] of the compute dtype; a k head also goes to its row of the
// cache, and its value head (the raw x with `v_from_k`, else the projection's own v head plus its bias) to
// the packed row and the cache.  `pitch` > 0 (>= hd and >= dv): the heads of the packed row and the rows of the
// cache are that many elements apart, zeros behind a head's own (a mixer pads its heads up to a size that the
// tensor-core attention kernels take); 0: q and k heads hd apart, v heads dv apart.
// Where a k head's row of token t goes in the cache (nullptr: nowhere).
template <typename T>
__device__ __forceinline__ void qk_cache_rows(T* kcache, T* vcache, const int* __restrict__ seq_of_token,
                                              const int* __restrict__ slots, const int* __restrict__ len_after,
                                              const int* __restrict__ page_table, int max_pages, int ring_rows, int nkv,
                                              int t, int pos, int g, int pk, int pv, T** kdst, T** vdst) {
  *kdst = nullptr, *vdst = nullptr;
  if (kcache == nullptr) return;
  const int seq = seq_of_token[t];
  const int slot = slots[seq];
  if (slot >= 0 && !(ring_rows > 0 && pos + ring_rows < len_after[seq])) {
    const int r = ring_rows > 0 ? pos % ring_rows : pos;
    if (AF_INDEX_OK(pos >= 0 && r / AF_PAGE < max_pages, r)) {
      const int page = page_table[(size_t)slot * max_pages + r / AF_PAGE];
      if (AF_INDEX_OK(page >= 0, page)) {
        const size_t at = ((size_t)page * nkv + g) * AF_PAGE + r % AF_PAGE;
        *kdst = kcache + at * pk;
        *vdst = vcache + at * pv;
      }
    }
  }
}

// One q or k head of one token, by one warp: norm (per head with the weight `w` of hd values, or with the factor
// `inv_whole` that the caller took over the whole projection and a weight that holds this head's own hd values),
// rotation, the norm behind it, packing, the cache row, and a k head's value head.
template <typename T>
__device__ __forceinline__ void qk_pack_head(T* __restrict__ qkv, long long out_stride, const float* __restrict__ proj,
                                             long long ld, const float* __restrict__ bias, const float* __restrict__ w,
                                             bool whole, float inv_whole, float eps, int norm_after, float magnitude,
                                             int v_from_k, const float* __restrict__ inv_freq,
                                             const float2* __restrict__ table, int nq, int nkv, int hd,
                                             int dv, int rot_dim, int pairing, int pk, int pv, int t, int head, int pos,
                                             int lane, T* kdst, T* vdst) {
  const bool is_k = head >= nq;
  const float* x = proj + (size_t)t * ld + (size_t)head * hd;
  const float* xb = bias ? bias + (size_t)head * hd : nullptr;
  T* orow = qkv + (size_t)t * out_stride;
  T* dst = orow + (size_t)head * pk;                        // q heads and k heads keep their places
  float inv = whole ? inv_whole : 1.f;
  if (w != nullptr && !whole) {
    float ss = 0.f;
    for (int i = lane; i < hd; i += 32) {
      const float v = x[i] + (xb ? xb[i] : 0.f);
      ss += v * v;
    }
    ss = warp_sum(ss);
    inv = rsqrtf(ss / (float)hd + eps);
  }
  float after = 1.f;
  if (norm_after) {
    // a rotation keeps a pair's length: the mean square after it is that of the rotated elements times
    // magnitude^2 plus that of the others
    float lo = 0.f, hi = 0.f;
    for (int i = lane; i < hd; i += 32) {
      float v = x[i] + (xb ? xb[i] : 0.f);
      if (w) v *= inv * w[i];
      if (i < rot_dim) lo += v * v; else hi += v * v;
    }
    lo = warp_sum(lo);
    hi = warp_sum(hi);
    after = rsqrtf((magnitude * magnitude * lo + hi) / (float)hd + eps);
  }
  const int half = rot_dim / 2;
  for (int p = lane; p < half; p += 32) {
    const int i0 = pairing == AF_PAIR_HALF ? p : 2 * p;
    const int i1 = pairing == AF_PAIR_HALF ? p + half : 2 * p + 1;
    float a = x[i0] + (xb ? xb[i0] : 0.f), b = x[i1] + (xb ? xb[i1] : 0.f);
    if (w) a *= inv * w[i0], b *= inv * w[i1];
    float s, c;
    if (table != nullptr) {                     // the step's table of (cos, sin) per token and pair
      const float2 cs = table[(size_t)t * half + p];
      c = cs.x, s = cs.y;
    } else {
      sincosf((float)pos * inv_freq[p], &s, &c);
    }
    s *= magnitude, c *= magnitude;
    const T ra = from_f32<T>((a * c - b * s) * after), rb = from_f32<T>((b * c + a * s) * after);
    dst[i0] = ra, dst[i1] = rb;
    if (kdst != nullptr) kdst[i0] = ra, kdst[i1] = rb;
  }
  for (int i = rot_dim + lane; i < hd; i += 32) {
    float a = x[i] + (xb ? xb[i] : 0.f);
    if (w) a *= inv * w[i];
    const T v = from_f32<T>(a * after);
    dst[i] = v;
    if (kdst != nullptr) kdst[i] = v;
  }
  for (int i = hd + lane; i < pk; i += 32) {                // the padding behind the head
    dst[i] = from_f32<T>(0.f);
    if (kdst != nullptr) kdst[i] = from_f32<T>(0.f);
  }
  if (is_k) {
    const int g = head - nq;
    const size_t v_off = (size_t)(nq + nkv) * hd + (size_t)g * dv;          // the value head's place in the projection
    const float* vx = v_from_k ? x : proj + (size_t)t * ld + v_off;
    const float* vb = bias == nullptr ? nullptr : (v_from_k ? xb : bias + v_off);
    T* vrow = orow + (size_t)(nq + nkv) * pk + (size_t)g * pv;              // and in the packed row
    for (int i = lane; i < pv; i += 32) {
      const T v = from_f32<T>(i < dv ? vx[i] + (vb && !v_from_k ? vb[i] : 0.f) : 0.f);
      vrow[i] = v;
      if (vdst != nullptr) vdst[i] = v;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
qk_norm_rope_store_kernel(T* __restrict__ qkv, long long out_stride, const float* __restrict__ proj, long long ld,
                          const float* __restrict__ bias, const float* __restrict__ q_weight,
                          const float* __restrict__ k_weight, float eps, int norm_after, float magnitude,
                          int v_from_k, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                          const int* __restrict__ slots, const int* __restrict__ len_after,
                          const float* __restrict__ inv_freq, const float2* __restrict__ table, int n_tokens, int nq,
                          int nkv, int hd, int dv, int rot_dim,
                          int pairing, T* __restrict__ kcache, T* __restrict__ vcache,
                          const int* __restrict__ page_table, int max_pages, int ring_rows, int pitch) {
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const long long wi = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wi >= (long long)n_tokens * (nq + nkv)) return;
  const int t = (int)(wi / (nq + nkv)), head = (int)(wi % (nq + nkv));
  const int pos = positions[t];
  const int pk = pitch > 0 ? pitch : hd, pv = pitch > 0 ? pitch : dv;      // elements between heads (and of a cache row)
  T *kdst = nullptr, *vdst = nullptr;
  if (head >= nq)
    qk_cache_rows(kcache, vcache, seq_of_token, slots, len_after, page_table, max_pages, ring_rows, nkv, t, pos,
                  head - nq, pk, pv, &kdst, &vdst);
  pdl_wait();
  qk_pack_head(qkv, out_stride, proj, ld, bias, head >= nq ? k_weight : q_weight, false, 1.f, eps, norm_after, magnitude,
               v_from_k, inv_freq, table, nq, nkv, hd, dv, rot_dim, pairing, pk, pv, t, head, pos, lane, kdst, vdst);
}

// The same with q (and k) normed over the whole projection of the token, all heads at once: the weights hold
// nq * hd and nkv * hd values.  One block per token: the two mean squares first, then a warp per head in turn.
template <typename T>
__global__ void __launch_bounds__(256)
qk_whole_norm_rope_store_kernel(T* __restrict__ qkv, long long out_stride, const float* __restrict__ proj, long long ld,
                                const float* __restrict__ bias, const float* __restrict__ q_weight,
                                const float* __restrict__ k_weight, float eps, int norm_after, float magnitude,
                                int v_from_k, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                const int* __restrict__ slots, const int* __restrict__ len_after,
                                const float* __restrict__ inv_freq, const float2* __restrict__ table, int nq, int nkv,
                                int hd, int dv, int rot_dim,
                                int pairing, T* __restrict__ kcache, T* __restrict__ vcache,
                                const int* __restrict__ page_table, int max_pages, int ring_rows, int pitch) {
  pdl_launch_dependents();
  __shared__ float scratch[33];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int pk = pitch > 0 ? pitch : hd, pv = pitch > 0 ? pitch : dv;
  pdl_wait();
  const float* row = proj + (size_t)t * ld;
  const int n_q = nq * hd, n_k = nkv * hd;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < n_q + n_k; i += blockDim.x) {
    const float v = row[i] + (bias ? bias[i] : 0.f);
    if (i < n_q) sq += v * v; else sk += v * v;
  }
  sq = block_sum(sq, scratch);
  sk = block_sum(sk, scratch);
  const float inv_q = rsqrtf(sq / (float)n_q + eps), inv_k = rsqrtf(sk / (float)n_k + eps);
  for (int head = warp; head < nq + nkv; head += nwarp) {
    const bool is_k = head >= nq;
    T *kdst = nullptr, *vdst = nullptr;
    if (is_k)
      qk_cache_rows(kcache, vcache, seq_of_token, slots, len_after, page_table, max_pages, ring_rows, nkv, t, pos,
                    head - nq, pk, pv, &kdst, &vdst);
    const float* w = is_k ? k_weight + (size_t)(head - nq) * hd : q_weight + (size_t)head * hd;
    qk_pack_head(qkv, out_stride, proj, ld, bias, w, true, is_k ? inv_k : inv_q, eps, norm_after, magnitude, v_from_k,
                 inv_freq, table, nq, nkv, hd, dv, rot_dim, pairing, pk, pv, t, head, pos, lane, kdst, vdst);
  }
}

// The same with the token's projection row in shared memory (rows of up to 12,288 values, the norm in front of the
// rotation, values of their own): the row is read once, both mean squares leave one reduction, the cache row is
// looked up once a token, and the pairs of all heads are one flat loop whose loads do not wait for one another.
template <typename T>
__global__ void __launch_bounds__(256)
qk_whole_norm_rope_row_kernel(T* __restrict__ qkv, long long out_stride, const float* __restrict__ proj, long long ld,
                              const float* __restrict__ bias, const float* __restrict__ q_weight,
                              const float* __restrict__ k_weight, float eps, float magnitude,
                              const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                              const int* __restrict__ slots, const int* __restrict__ len_after,
                              const float* __restrict__ inv_freq, const float2* __restrict__ table, int nq, int nkv,
                              int hd, int dv, int rot_dim, int pairing, T* __restrict__ kcache, T* __restrict__ vcache,
                              const int* __restrict__ page_table, int max_pages, int ring_rows, int pitch) {
  pdl_launch_dependents();
  extern __shared__ __align__(16) float srow[];          // q | k | v of the token, biases added
  __shared__ float red[2][8];
  __shared__ T* cache_rows[2];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int pk = pitch > 0 ? pitch : hd, pv = pitch > 0 ? pitch : dv;
  if (threadIdx.x == 0) {                                // (the step's tables are there before the step begins)
    T *k0 = nullptr, *v0 = nullptr;
    qk_cache_rows(kcache, vcache, seq_of_token, slots, len_after, page_table, max_pages, ring_rows, nkv, t, pos, 0, pk,
                  pv, &k0, &v0);
    cache_rows[0] = k0, cache_rows[1] = v0;
  }
  pdl_wait();
  const float* row = proj + (size_t)t * ld;
  const int n_q = nq * hd, n_k = nkv * hd, n_all = n_q + n_k + nkv * dv;
  float sq = 0.f, sk = 0.f;
#pragma unroll 4
  for (int i = threadIdx.x; i < n_all; i += 256) {
    const float v = row[i] + (bias ? bias[i] : 0.f);
    srow[i] = v;
    if (i < n_q) sq += v * v; else if (i < n_q + n_k) sk += v * v;
  }
  sq = warp_sum(sq), sk = warp_sum(sk);
  if (lane == 0) red[0][warp] = sq, red[1][warp] = sk;
  __syncthreads();
  sq = sk = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) sq += red[0][w], sk += red[1][w];
  const float inv_q = rsqrtf(sq / (float)n_q + eps), inv_k = rsqrtf(sk / (float)n_k + eps);
  T* orow = qkv + (size_t)t * out_stride;
  T* kd0 = cache_rows[0];
  T* vd0 = cache_rows[1];
  const int heads = nq + nkv, half = rot_dim / 2;
  // (q weights and k weights: heads x hd values each, in the heads' order)
  for (int idx = threadIdx.x; idx < heads * half; idx += 256) {
    const int head = idx / half, p = idx % half;
    const bool is_k = head >= nq;
    const int i0 = pairing == AF_PAIR_HALF ? p : 2 * p, i1 = pairing == AF_PAIR_HALF ? p + half : 2 * p + 1;
    const float* w = is_k ? k_weight + (size_t)(head - nq) * hd : q_weight + (size_t)head * hd;
    const float inv = is_k ? inv_k : inv_q;
    const float a = srow[head * hd + i0] * inv * w[i0], b = srow[head * hd + i1] * inv * w[i1];
    float s, c;
    if (table != nullptr) {
      const float2 cs = table[(size_t)t * half + p];
      c = cs.x, s = cs.y;
    } else {
      sincosf((float)pos * inv_freq[p], &s, &c);
    }
    s *= magnitude, c *= magnitude;
    const T ra = from_f32<T>(a * c - b * s), rb = from_f32<T>(b * c + a * s);
    T* dst = orow + (size_t)head * pk;
    dst[i0] = ra, dst[i1] = rb;
    if (is_k && kd0 != nullptr) {
      T* kdst = kd0 + (size_t)(head - nq) * AF_PAGE * pk;
      kdst[i0] = ra, kdst[i1] = rb;
    }
  }
  const int rest = pk - rot_dim;                         // behind the rotated part: kept elements, then padding
  for (int idx = threadIdx.x; idx < heads * rest; idx += 256) {
    const int head = idx / rest, i = rot_dim + idx % rest;
    const bool is_k = head >= nq;
    float v = 0.f;
    if (i < hd) {
      const float* w = is_k ? k_weight + (size_t)(head - nq) * hd : q_weight + (size_t)head * hd;
      v = srow[head * hd + i] * (is_k ? inv_k : inv_q) * w[i];
    }
    const T r = from_f32<T>(v);
    orow[(size_t)head * pk + i] = r;
    if (is_k && kd0 != nullptr) kd0[(size_t)(head - nq) * AF_PAGE * pk + i] = r;
  }
  T* vrow = orow + (size_t)heads * pk;
  for (int idx = threadIdx.x; idx < nkv * pv; idx += 256) {
    const int g = idx / pv, i = idx % pv;
    const T r = from_f32<T>(i < dv ? srow[n_q + n_k + g * dv + i] : 0.f);
    vrow[(size_t)g * pv + i] = r;
    if (vd0 != nullptr) vd0[(size_t)g * AF_PAGE * pv + i] = r;
  }
}

AF_EXPORT int af_qk_norm_rope_store(void* qkv, int dtype, long long out_stride, const float* proj, long long ld,
                                    const float* bias, const float* q_weight, const float* k_weight, float eps,
                                    int norm_after, float magnitude, int v_from_k,
                                    const int* positions, const int* seq_of_token, const int* slots,
                                    const int* len_after, const float* inv_freq, const float* table, int n_tokens,
                                    int nq, int nkv, int hd,
                                    int dv, int rot_dim, int pairing, void* kcache, void* vcache, const int* page_table,
                                    int max_pages, int ring_rows, int pitch, int whole_norm, cudaStream_t stream) {
  const float2* tab = reinterpret_cast<const float2*>(table);
  AF_REQUIRE(((uintptr_t)table & 7) == 0, "af_qk_norm_rope_store: the table of cosines and sines lies on 8 bytes");
  if (n_tokens == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && nq > 0 && nkv > 0 && hd > 0 && dv > 0, "af_qk_norm_rope_store: bad sizes");
  AF_REQUIRE(!whole_norm || q_weight != nullptr, "af_qk_norm_rope_store: a norm over the whole projection needs its weights");
  AF_REQUIRE(pitch == 0 || (pitch >= hd && pitch >= dv), "af_qk_norm_rope_store: pitch %d below the heads' sizes", pitch);

  AF_REQUIRE(!v_from_k || dv == hd, "af_qk_norm_rope_store: values that are the keys have their size");
  AF_REQUIRE(rot_dim >= 0 && rot_dim <= hd && rot_dim % 2 == 0,
             "af_qk_norm_rope_store: rotary dim %d must be even and <= head_dim %d", rot_dim, hd);
  AF_REQUIRE(pairing == AF_PAIR_HALF || pairing == AF_PAIR_ADJACENT, "af_qk_norm_rope_store: pairing");
  AF_REQUIRE(ring_rows % AF_PAGE == 0, "af_qk_norm_rope_store: ring rows %d not whole pages", ring_rows);
  AF_REQUIRE((kcache == nullptr) == (vcache == nullptr), "af_qk_norm_rope_store: k and v cache");
  AF_REQUIRE((q_weight == nullptr) == (k_weight == nullptr), "af_qk_norm_rope_store: both norm weights or none");
  const size_t row_bytes = ((size_t)(nq + nkv) * hd + (size_t)nkv * dv) * sizeof(float);
  if (whole_norm && !norm_after && !v_from_k && row_bytes <= 48 * 1024) {
    AF_DISPATCH_DTYPE(dtype, T,
                      af_launch(qk_whole_norm_rope_row_kernel<T>, dim3((unsigned)n_tokens), dim3(256), row_bytes, stream,
                                (T*)qkv, out_stride, proj, ld, bias, q_weight, k_weight, eps, magnitude, positions,
                                seq_of_token, slots, len_after, inv_freq, tab, nq, nkv, hd, dv, rot_dim, pairing,
                                (T*)kcache, (T*)vcache, page_table, max_pages, ring_rows, pitch));
    AF_CHECK_LAUNCH("af_qk_norm_rope_store");
  }
  if (whole_norm) {
    AF_DISPATCH_DTYPE(dtype, T,
                      af_launch(qk_whole_norm_rope_store_kernel<T>, dim3((unsigned)n_tokens), dim3(256), 0, stream, (T*)qkv,
                                out_stride, proj, ld, bias, q_weight, k_weight, eps, norm_after, magnitude, v_from_k,
                                positions, seq_of_token, slots, len_after, inv_freq, tab, nq, nkv, hd, dv, rot_dim, pairing,
                                (T*)kcache, (T*)vcache, page_table, max_pages, ring_rows, pitch));
    AF_CHECK_LAUNCH("af_qk_norm_rope_store");
  }
  const long long warps = (long long)n_tokens * (nq + nkv);
  const long long blocks = (warps + 3) / 4;
  AF_REQUIRE(blocks < (1ll << 31), "af_qk_norm_rope_store: too many rows");
  AF_DISPATCH_DTYPE(dtype, T,
                    af_launch(qk_norm_rope_store_kernel<T>, dim3((unsigned)blocks), dim3(128), 0, stream, (T*)qkv,
                              out_stride, proj, ld, bias, q_weight, k_weight, eps, norm_after, magnitude, v_from_k,
                              positions, seq_of_token, slots, len_after, inv_freq, tab, n_tokens, nq, nkv, hd, dv, rot_dim,
                              pairing, (T*)kcache, (T*)vcache, page_table, max_pages, ring_rows, pitch));
  AF_CHECK_LAUNCH("af_qk_norm_rope_store");
}

// ---------------------------------------------------------------- keys and values from a latent vector

// From float projection rows [q heads of (dim + rot) | latent of `rank` | shared key part of `rot`]:
//   q heads: the last `rot` elements of every head rotated (pairs i, i + rot / 2), the first `dim` kept,
//            into the rows `q` of the compute dtype, head u at u * pitch (pitch >= dim + rot; the elements
//            between a head's end and the next head's start are set to zero);
//   the latent divided by its root mean square (eps inside the root) times `norm_w`, and the shared key
//   part rotated, into the row `kv` [rank + rot] of the compute dtype and into the token's row of its cache
//   page (one kv head of rank + rot elements; the values are the latent part of the same row).
// One block per token.
template <typename T>
__global__ void __launch_bounds__(256)
latent_prep_kernel(T* __restrict__ q, long long q_stride, T* __restrict__ kv, long long kv_stride,
                   const float* __restrict__ proj, long long ld, const float* __restrict__ norm_w, float eps,
                   const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                   const int* __restrict__ slots, const int* __restrict__ len_after,
                   const float* __restrict__ inv_freq, int heads, int dim, int rot, int rank, int pitch,
                   T* __restrict__ kcache, const int* __restrict__ page_table, int max_pages, int ring_rows) {
  pdl_launch_dependents();
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int width = rank + rot;
  T* kdst = nullptr;
  if (kcache != nullptr) {
    const int seq = seq_of_token[t];
    const int slot = slots[seq];
    if (slot >= 0 && !(ring_rows > 0 && pos + ring_rows < len_after[seq])) {
      const int r = ring_rows > 0 ? pos % ring_rows : pos;
      if (AF_INDEX_OK(pos >= 0 && r / AF_PAGE < max_pages, r)) {
        const int page = page_table[(size_t)slot * max_pages + r / AF_PAGE];
        if (AF_INDEX_OK(page >= 0, page)) kdst = kcache + ((size_t)page * AF_PAGE + r % AF_PAGE) * width;
      }
    }
  }
  pdl_wait();
  const float* x = proj + (size_t)t * ld;
  const float* lat = x + (size_t)heads * (dim + rot);
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) ss += lat[i] * lat[i];
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)rank + eps);
  T* kvr = kv + (size_t)t * kv_stride;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const T v = from_f32<T>(lat[i] * inv * norm_w[i]);
    kvr[i] = v;
    if (kdst != nullptr) kdst[i] = v;
  }
  const int half = rot / 2;
  T* qr = q + (size_t)t * q_stride;
  // rotated pairs: unit heads + 1 is the shared key part
  for (int i = threadIdx.x; i < (heads + 1) * half; i += blockDim.x) {
    const int u = i / half, p = i - u * half;
    float s, c;
    sincosf((float)pos * inv_freq[p], &s, &c);
    const float* src = u < heads ? x + (size_t)u * (dim + rot) + dim : lat + rank;
    const float a = src[p], b = src[p + half];
    const T ra = from_f32<T>(a * c - b * s), rb = from_f32<T>(b * c + a * s);
    if (u < heads) {
      T* d = qr + (size_t)u * pitch + dim;
      d[p] = ra, d[p + half] = rb;
    } else {
      kvr[rank + p] = ra, kvr[rank + p + half] = rb;
      if (kdst != nullptr) kdst[rank + p] = ra, kdst[rank + p + half] = rb;
    }
  }
  for (int i = threadIdx.x; i < heads * dim; i += blockDim.x) {
    const int u = i / dim, e = i - u * dim;
    qr[(size_t)u * pitch + e] = from_f32<T>(x[(size_t)u * (dim + rot) + e]);
  }
  const int pad = pitch - dim - rot;
  for (int i = threadIdx.x; i < heads * pad; i += blockDim.x) {
    const int u = i / pad, e = i - u * pad;
    qr[(size_t)u * pitch + dim + rot + e] = from_f32<T>(0.f);
  }
}

AF_EXPORT int af_latent_prep(void* q, long long q_stride, void* kv, long long kv_stride, int dtype, const float* proj,
                             long long ld, const float* norm_w, float eps, const int* positions,
                             const int* seq_of_token, const int* slots, const int* len_after, const float* inv_freq,
                             int n_tokens, int heads, int dim, int rot, int rank, int pitch, void* kcache,
                             const int* page_table, int max_pages, int ring_rows, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && heads > 0 && dim >= 0 && rot >= 0 && rot % 2 == 0 && rank > 0 && dim + rot > 0 &&
             pitch >= dim + rot, "af_latent_prep: bad sizes");
  AF_REQUIRE(ring_rows % AF_PAGE == 0, "af_latent_prep: ring rows %d not whole pages", ring_rows);
  AF_DISPATCH_DTYPE(dtype, T,
                    af_launch(latent_prep_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, (T*)q, q_stride, (T*)kv,
                              kv_stride, proj, ld, norm_w, eps, positions, seq_of_token, slots, len_after, inv_freq,
                              heads, dim, rot, rank, pitch, (T*)kcache, page_table, max_pages, ring_rows));
  AF_CHECK_LAUNCH("af_latent_prep");
}

// ---------------------------------------------------------------- a small product per head

// out[t, h, n] = sum_d x[t, h, d] * w[h, d, n] for d < D, n < N (32-bit sums), and the
// `extra` elements that follow a head's D inputs copied behind its N outputs.  x rows: heads `x_pitch`
// elements apart (at least D + extra), rows `x_stride` apart; out rows: heads of (N + extra), `out_stride` apart;
// w [heads, D, N].
// One block of 256 threads per (token, head); the head's inputs wait in shared memory.  With fewer than 256
// outputs the threads form 256 / cols groups that each take a stretch of the inputs (a long sum is then several
// short chains side by side); the groups' sums are added in group order.
template <typename T>
__global__ void __launch_bounds__(256)
head_project_kernel(T* __restrict__ out, long long out_stride, const T* __restrict__ x, long long x_stride,
                    const T* __restrict__ w, int D, int N, int extra, int x_pitch, int cols) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float xs[];                     // D inputs, then [groups][cols] partial sums
  float* red = xs + D;
  const int t = blockIdx.x, h = blockIdx.y;
  const T* xr = x + (size_t)t * x_stride + (size_t)h * x_pitch;
  T* o = out + (size_t)t * out_stride + (size_t)h * (N + extra);
  for (int d = threadIdx.x; d < D; d += blockDim.x) xs[d] = to_f32(xr[d]);
  for (int e = threadIdx.x; e < extra; e += blockDim.x) o[N + e] = xr[D + e];
  __syncthreads();
  const T* wh = w + (size_t)h * D * N;
  const int groups = blockDim.x / cols, grp = threadIdx.x / cols, col = threadIdx.x - grp * cols;
  const int per = (D + groups - 1) / groups, d0 = grp * per, d1 = min(D, d0 + per);
  for (int n0 = 0; n0 < N; n0 += cols) {            // (several rounds only when there is one group)
    const int n = n0 + col;
    float acc = 0.f;
    if (n < N && grp < groups) {
#pragma unroll 8
      for (int d = d0; d < d1; ++d) acc += xs[d] * to_f32(wh[(size_t)d * N + n]);
    }
    if (groups == 1) {
      if (n < N) o[n] = from_f32<T>(acc);
      continue;
    }
    if (grp < groups) red[grp * cols + col] = acc;
    __syncthreads();
    if (grp == 0 && n < N) {
      float sum = red[col];
      for (int g2 = 1; g2 < groups; ++g2) sum += red[g2 * cols + col];
      o[n] = from_f32<T>(sum);
    }
  }
}

// The same for the few rows of a decode step: a block takes 32 outputs of a head for eight tokens at once, so a
// weight is read once for all of them; its 256 threads are 8 groups that each take a stretch of the inputs
// (short chains side by side), joined in group order through shared memory.  Grid (head, 32 outputs, 8 tokens).
template <typename T>
__global__ void __launch_bounds__(256)
head_project_few_kernel(T* __restrict__ out, long long out_stride, const T* __restrict__ x, long long x_stride,
                        const T* __restrict__ w, int D, int N, int extra, int x_pitch, int n_tokens) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float xs[];                     // [8 tokens][D] inputs, then [8 groups][8 tokens][32] partial sums
  float* red = xs + 8 * D;
  const int h = blockIdx.x, n = blockIdx.y * 32 + (threadIdx.x & 31), t0 = blockIdx.z * 8;
  const int grp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 8 * D; i += blockDim.x) {
    const int u = i / D, d = i - u * D;
    xs[i] = t0 + u < n_tokens ? to_f32(x[(size_t)(t0 + u) * x_stride + (size_t)h * x_pitch + d]) : 0.f;
  }
  if (blockIdx.y == 0)
    for (int i = threadIdx.x; i < 8 * extra; i += blockDim.x) {
      const int u = i / extra, e = i - u * extra;
      if (t0 + u < n_tokens)
        out[(size_t)(t0 + u) * out_stride + (size_t)h * (N + extra) + N + e] = x[(size_t)(t0 + u) * x_stride + (size_t)h * x_pitch + D + e];
    }
  __syncthreads();
  const int per = (D + 7) / 8, d0 = grp * per, d1 = min(D, d0 + per);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (n < N) {
    const T* wh = w + (size_t)h * D * N + n;
#pragma unroll 4
    for (int d = d0; d < d1; ++d) {
      const float wv = to_f32(wh[(size_t)d * N]);
#pragma unroll
      for (int u = 0; u < 8; ++u) acc[u] += xs[u * D + d] * wv;
    }
  }
#pragma unroll
  for (int u = 0; u < 8; ++u) red[(grp * 8 + u) * 32 + (threadIdx.x & 31)] = acc[u];
  __syncthreads();
  const int u = threadIdx.x >> 5;                   // (now: the token this thread writes)
  if (n < N && t0 + u < n_tokens) {
    float sum = 0.f;
#pragma unroll
    for (int g2 = 0; g2 < 8; ++g2) sum += red[(g2 * 8 + u) * 32 + (threadIdx.x & 31)];
    out[(size_t)(t0 + u) * out_stride + (size_t)h * (N + extra) + n] = from_f32<T>(sum);
  }
}

AF_EXPORT int af_head_project(void* out, long long out_stride, const void* x, long long x_stride, const void* w,
                              int dtype, int n_tokens, int heads, int D, int N, int extra, int x_pitch,
                              cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && heads > 0 && heads < 65536 && D > 0 && N > 0 && extra >= 0 && x_pitch >= D + extra,
             "af_head_project: bad sizes");
  AF_REQUIRE((size_t)(D + 256) * sizeof(float) <= 48 * 1024, "af_head_project: %d inputs a head beyond 12032", D);
  if (n_tokens <= 64 && (size_t)(8 * D + 2048) * sizeof(float) <= 48 * 1024 && (N + 31) / 32 < 65536) {
    AF_DISPATCH_DTYPE(dtype, T,
                      af_launch(head_project_few_kernel<T>, dim3(heads, (N + 31) / 32, (n_tokens + 7) / 8), dim3(256),
                                (size_t)(8 * D + 2048) * sizeof(float), stream, (T*)out, out_stride, (const T*)x, x_stride,
                                (const T*)w, D, N, extra, x_pitch, n_tokens));
    AF_CHECK_LAUNCH("af_head_project");
  }
  const int cols = N >= 256 ? 256 : ((N + 31) / 32) * 32;          // outputs a round; 256 / cols groups share the inputs
  AF_DISPATCH_DTYPE(dtype, T,
                    af_launch(head_project_kernel<T>, dim3(n_tokens, heads), dim3(256), (size_t)(D + 256) * sizeof(float),
                              stream, (T*)out, out_stride, (const T*)x, x_stride, (const T*)w, D, N, extra, x_pitch, cols));
  AF_CHECK_LAUNCH("af_head_project");
}
