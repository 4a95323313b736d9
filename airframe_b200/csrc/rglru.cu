// A gated linear recurrence over a vector state with a short causal convolution in front (the recurrent block
// of Griffin: De et al., "Griffin: Mixing Gated Linear Recurrences with Local Attention for Efficient Language
// Models"), in three kernels between the input and output products:
//   conv_rows   u = conv(x + bx) + cb per channel over the tokens of each sequence, the tokens before the step
//               taken from the sequence's state;
//   gate_rows   r = sigmoid(Wa_b u_b + ba), i = sigmoid(Wi_b u_b + bi) with block-diagonal Wa, Wi (b = the
//               block of channels), then a = exp(-c r softplus(lam)) and the token's input sqrt(1 - a^2) i u;
//               what is kept of a is 1 - a = -expm1(log a): a itself, rounded to 32 bits next to 1, would lose
//               most of the bits that say how fast a slow channel forgets;
//   decay_scan  S <- a S + input = S - (1 - a) S + input token after token, out = S * gelu_tanh(y + by), and the state left for the next
//               step: S and the last taps - 1 inputs of the convolution.
// Everything here is 32-bit: the rows come from products that accumulate in 32 bits, the weights of the gates are
// read in the compute dtype and widened, and only the output (the input of the output product) is of the compute dtype.
// The state of a sequence is float [taps][width]: row 0 is S, rows 1 .. taps-1 the convolution's last inputs, oldest first.
#include "common.cuh"

// ---------------------------------------------------------------- the convolution

__global__ void __launch_bounds__(256)
conv_rows_kernel(float* __restrict__ u, __nv_bfloat16* __restrict__ u16, const float* __restrict__ proj, long long ld, int off_x,
                 const float* __restrict__ bx, const float* __restrict__ cw, const float* __restrict__ cb,
                 const float* __restrict__ state, const int* __restrict__ seq_of_token,
                 const int* __restrict__ seq_starts, const int* __restrict__ slots, int n_tokens, int width, int taps) {
  pdl_launch_dependents();
  // (a block: 256 channels of one token; no division a value)
  const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= width) return;
  const size_t i = (size_t)t * width + c;
  const int seq = seq_of_token[t];
  const int first = seq_starts[seq];
  const int slot = slots[seq];
  const float xb = bx[c];
  float acc = cb[c];
  pdl_wait();
  proj = pdl_fresh(proj);
  state = pdl_fresh(state);
  for (int k = 0; k < taps; ++k) {
    const int src = t - (taps - 1 - k);             // the token this tap looks at (the last tap: the current one)
    float v;
    if (src >= first) {
      v = proj[(size_t)src * ld + off_x + c] + xb;
    } else {
      // before the step: row 1 + (taps - 1) + (src - first) of the state (zeros for a sequence that just began)
      v = slot >= 0 ? state[((size_t)slot * taps + (taps + src - first)) * width + c] : 0.f;
    }
    acc += cw[(size_t)k * width + c] * v;           // (taps stored [taps, width]: a warp reads one line)
  }
  u[i] = acc;
  if (u16 != nullptr) u16[i] = __float2bfloat16_rn(acc);      // (what a tensor-core product of the gates reads)
}

// Up to eight taps: a thread takes one channel of four consecutive tokens.  The inputs of its window are asked for
// before it knows where the tokens' sequences begin (the tables' loads and the window's run side by side, and a
// value is read once for the four tokens); a tap that reaches before a sequence's first token of the step takes
// the slot's history instead.  Every output adds its taps from the oldest to the newest.
#define AF_CV_TOKENS 4
#define AF_CV_TAPS 8
__global__ void __launch_bounds__(256)
conv_rows_window_kernel(float* __restrict__ u, __nv_bfloat16* __restrict__ u16, const float* __restrict__ proj,
                        long long ld, int off_x, const float* __restrict__ bx, const float* __restrict__ cw,
                        const float* __restrict__ cb, const float* __restrict__ state,
                        const int* __restrict__ seq_of_token, const int* __restrict__ seq_starts,
                        const int* __restrict__ slots, int n_tokens, int width, int taps) {
  pdl_launch_dependents();
  const int t0 = blockIdx.x * AF_CV_TOKENS, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= width) return;
  int first[AF_CV_TOKENS], slot[AF_CV_TOKENS];
#pragma unroll
  for (int e = 0; e < AF_CV_TOKENS; ++e) {
    const int seq = t0 + e < n_tokens ? seq_of_token[t0 + e] : -1;
    first[e] = seq >= 0 ? seq_starts[seq] : 0;
    slot[e] = seq >= 0 ? slots[seq] : -1;
  }
  const float xb = bx[c], bias = cb[c];
  float tap[AF_CV_TAPS];                              // tap[d]: the weight on the token d back
#pragma unroll
  for (int d = 0; d < AF_CV_TAPS; ++d) tap[d] = d < taps ? cw[(size_t)(taps - 1 - d) * width + c] : 0.f;
  pdl_wait();
  proj = pdl_fresh(proj);
  state = pdl_fresh(state);
  float win[AF_CV_TOKENS + AF_CV_TAPS - 1];           // win[j]: the input of token t0 - (AF_CV_TAPS - 1) + j
#pragma unroll
  for (int j = 0; j < AF_CV_TOKENS + AF_CV_TAPS - 1; ++j) {
    const int src = t0 - (AF_CV_TAPS - 1) + j;
    win[j] = (j >= AF_CV_TAPS - taps && src >= 0 && src < n_tokens) ? proj[(size_t)src * ld + off_x + c] + xb : 0.f;
  }
#pragma unroll
  for (int e = 0; e < AF_CV_TOKENS; ++e) {
    const int t = t0 + e;
    if (t >= n_tokens) break;
    float acc = bias;
#pragma unroll
    for (int d = AF_CV_TAPS - 1; d >= 0; --d) {
      if (d >= taps) continue;
      const int src = t - d;
      float v = win[AF_CV_TAPS - 1 + e - d];
      if (src < first[e])                             // before the step: the slot's history (zeros for a new sequence)
        v = slot[e] >= 0 ? state[((size_t)slot[e] * taps + (taps + src - first[e])) * width + c] : 0.f;
      acc += tap[d] * v;
    }
    const size_t i = (size_t)t * width + c;
    u[i] = acc;
    if (u16 != nullptr) u16[i] = __float2bfloat16_rn(acc);
  }
}

AF_EXPORT int af_conv_rows(float* u, void* u16, const float* proj, long long ld, int off_x, const float* bx, const float* cw,
                           const float* cb, const float* state, const int* seq_of_token, const int* seq_starts,
                           const int* slots, int n_tokens, int width, int taps, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && width > 0 && taps >= 1, "af_conv_rows: bad sizes");
  const int chunks = (width + 255) / 256;
  AF_REQUIRE(chunks < 65536, "af_conv_rows: too many channels");
  // (a decode step's few tokens each begin in their slot's history: a value a thread serves them better)
  if (taps <= AF_CV_TAPS && n_tokens >= 64) {
    af_launch(conv_rows_window_kernel, dim3((unsigned)((n_tokens + AF_CV_TOKENS - 1) / AF_CV_TOKENS), (unsigned)chunks),
              dim3(256), 0, stream, u, (__nv_bfloat16*)u16, proj, ld, off_x, bx, cw, cb, state, seq_of_token, seq_starts,
              slots, n_tokens, width, taps);
    AF_CHECK_LAUNCH("af_conv_rows");
  }
  af_launch(conv_rows_kernel, dim3((unsigned)n_tokens, (unsigned)chunks), dim3(256), 0, stream, u, (__nv_bfloat16*)u16, proj, ld, off_x, bx, cw, cb, state,
            seq_of_token, seq_starts, slots, n_tokens, width, taps);
  AF_CHECK_LAUNCH("af_conv_rows");
}

// ---------------------------------------------------------------- the gates

// A block owns 32 tokens, one block of channels and 64 of its outputs, for both gates; thread (tx, ty) owns
// output tx for the tokens ty, ty + 4, ...  Every output adds its products in index order, whatever else is in
// the step.  Wa, Wi: [blocks][out][in] of the compute dtype.
#define AF_GR_TM 32
#define AF_GR_TN 64
#define AF_GR_TK 32
template <typename TW>
__global__ void __launch_bounds__(256)
gate_rows_kernel(float* __restrict__ decay, float* __restrict__ input, const float* __restrict__ u,
                 const TW* __restrict__ wa, const TW* __restrict__ wi, const float* __restrict__ ba,
                 const float* __restrict__ bi, const float* __restrict__ rate, int n_tokens, int width, int bw) {
  pdl_launch_dependents();
  __shared__ float us[AF_GR_TM][AF_GR_TK];
  __shared__ float was[AF_GR_TN][AF_GR_TK + 1];
  __shared__ float wis[AF_GR_TN][AF_GR_TK + 1];
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  const int t0 = blockIdx.x * AF_GR_TM, b = blockIdx.y, n0 = blockIdx.z * AF_GR_TN;
  const TW* wab = wa + (size_t)b * bw * bw;
  const TW* wib = wi + (size_t)b * bw * bw;
  float acc_a[AF_GR_TM / 4], acc_i[AF_GR_TM / 4];
#pragma unroll
  for (int m = 0; m < AF_GR_TM / 4; ++m) acc_a[m] = acc_i[m] = 0.f;
  pdl_wait();
  u = pdl_fresh(u);
  for (int k0 = 0; k0 < bw; k0 += AF_GR_TK) {
    for (int e = threadIdx.x; e < AF_GR_TM * AF_GR_TK; e += 256) {
      const int m = e / AF_GR_TK, k = e % AF_GR_TK;
      us[m][k] = (t0 + m < n_tokens && k0 + k < bw) ? u[(size_t)(t0 + m) * width + (size_t)b * bw + k0 + k] : 0.f;
    }
    for (int e = threadIdx.x; e < AF_GR_TN * AF_GR_TK; e += 256) {
      const int n = e / AF_GR_TK, k = e % AF_GR_TK;
      const bool in = n0 + n < bw && k0 + k < bw;
      was[n][k] = in ? to_f32<TW>(wab[(size_t)(n0 + n) * bw + k0 + k]) : 0.f;
      wis[n][k] = in ? to_f32<TW>(wib[(size_t)(n0 + n) * bw + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < AF_GR_TK; ++k) {
      const float a = was[tx][k], g = wis[tx][k];
#pragma unroll
      for (int m = 0; m < AF_GR_TM / 4; ++m) {
        const float v = us[ty + 4 * m][k];
        acc_a[m] = fmaf(a, v, acc_a[m]);
        acc_i[m] = fmaf(g, v, acc_i[m]);
      }
    }
    __syncthreads();
  }
  if (n0 + tx >= bw) return;
  const int c = b * bw + n0 + tx;
  const float ab = ba[c], ib = bi[c], rt = rate[c];
#pragma unroll
  for (int m = 0; m < AF_GR_TM / 4; ++m) {
    const int t = t0 + ty + 4 * m;
    if (t >= n_tokens) continue;
    const float r = 1.f / (1.f + expf(-(acc_a[m] + ab)));
    const float g = 1.f / (1.f + expf(-(acc_i[m] + ib)));
    const float la = -rt * r;                               // log a
    const size_t at = (size_t)t * width + c;
    decay[at] = -expm1f(la);                                // 1 - a
    input[at] = sqrtf(fmaxf(-expm1f(2.f * la), 0.f)) * g * u[at];      // sqrt(1 - a^2) i u
  }
}

// Few tokens (a decode step): a warp owns one output of both gates for eight tokens, whose u of this block of
// channels waits in shared memory; a lane reads eight weights of each matrix at a time.  Every output adds its
// products in an order that depends on nothing else in the step.
#define AF_GF_TM 8
template <typename TW>
__device__ __forceinline__ void load8_f32(float* v, const TW* p);
template <>
__device__ __forceinline__ void load8_f32<float>(float* v, const float* p) {
  const float4 t0 = *reinterpret_cast<const float4*>(p), t1 = *reinterpret_cast<const float4*>(p + 4);
  v[0] = t0.x, v[1] = t0.y, v[2] = t0.z, v[3] = t0.w, v[4] = t1.x, v[5] = t1.y, v[6] = t1.z, v[7] = t1.w;
}
template <>
__device__ __forceinline__ void load8_f32<__nv_bfloat16>(float* v, const __nv_bfloat16* p) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const unsigned r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) v[2 * j] = __uint_as_float(r[j] << 16), v[2 * j + 1] = __uint_as_float(r[j] & 0xffff0000u);
}

template <typename TW>
__global__ void __launch_bounds__(256)
gate_rows_few_kernel(float* __restrict__ decay, float* __restrict__ input, const float* __restrict__ u,
                     const TW* __restrict__ wa, const TW* __restrict__ wi, const float* __restrict__ ba,
                     const float* __restrict__ bi, const float* __restrict__ rate, int n_tokens, int width, int bw) {
  pdl_launch_dependents();
  extern __shared__ __align__(16) float uf[];               // [AF_GF_TM][bw]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n = blockIdx.x * 8 + warp, b = blockIdx.y, t0 = blockIdx.z * AF_GF_TM;
  const bool mine = n < bw;
  const TW* war = wa + ((size_t)b * bw + (mine ? n : 0)) * bw;
  const TW* wir = wi + ((size_t)b * bw + (mine ? n : 0)) * bw;
  // (the weights do not depend on the kernel in front: the first of them are on their way during the wait)
  float a8[8], g8[8];
  const int k_first = lane * 8;
  if (mine && k_first < bw) load8_f32<TW>(a8, war + k_first), load8_f32<TW>(g8, wir + k_first);
  pdl_wait();
  u = pdl_fresh(u);
  for (int e = threadIdx.x * 4; e < AF_GF_TM * bw; e += 1024) {
    const int m = e / bw, k = e % bw;                       // (bw is a multiple of 8: four values stay in a row)
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (t0 + m < n_tokens) v = *reinterpret_cast<const float4*>(u + (size_t)(t0 + m) * width + (size_t)b * bw + k);
    *reinterpret_cast<float4*>(uf + e) = v;
  }
  __syncthreads();
  if (!mine) return;
  float acc_a[AF_GF_TM], acc_i[AF_GF_TM];
#pragma unroll
  for (int m = 0; m < AF_GF_TM; ++m) acc_a[m] = acc_i[m] = 0.f;
  for (int k0 = k_first; k0 < bw; k0 += 256) {
    if (k0 != k_first) load8_f32<TW>(a8, war + k0), load8_f32<TW>(g8, wir + k0);
#pragma unroll
    for (int m = 0; m < AF_GF_TM; ++m) {
      const float4 v0 = *reinterpret_cast<const float4*>(uf + m * bw + k0);
      const float4 v1 = *reinterpret_cast<const float4*>(uf + m * bw + k0 + 4);
      const float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) acc_a[m] = fmaf(a8[j], v[j], acc_a[m]), acc_i[m] = fmaf(g8[j], v[j], acc_i[m]);
    }
  }
  float sa = 0.f, si = 0.f;                                 // lane m keeps token t0 + m's sums
#pragma unroll
  for (int m = 0; m < AF_GF_TM; ++m) {
    const float ta = warp_sum(acc_a[m]), ti = warp_sum(acc_i[m]);
    if (lane == m) sa = ta, si = ti;
  }
  const int t = t0 + lane;
  if (lane >= AF_GF_TM || t >= n_tokens) return;
  const int c = b * bw + n;
  const float r = 1.f / (1.f + expf(-(sa + ba[c])));
  const float g = 1.f / (1.f + expf(-(si + bi[c])));
  const float la = -rate[c] * r;                            // log a
  const size_t at = (size_t)t * width + c;
  decay[at] = -expm1f(la);                                  // 1 - a
  input[at] = sqrtf(fmaxf(-expm1f(2.f * la), 0.f)) * g * uf[lane * bw + n];      // sqrt(1 - a^2) i u
}

AF_EXPORT int af_gate_rows(float* decay, float* input, const float* u, const void* wa, const void* wi, int w_dtype,
                           const float* ba, const float* bi, const float* rate, int n_tokens, int width, int blocks,
                           cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && width > 0 && blocks > 0 && width % blocks == 0,
             "af_gate_rows: %d channels in %d blocks", width, blocks);
  const int bw = width / blocks;
  if (n_tokens <= 4 * AF_GF_TM && bw % 8 == 0 && (size_t)AF_GF_TM * bw * sizeof(float) <= 48 * 1024 &&
      (((uintptr_t)u | (uintptr_t)wa | (uintptr_t)wi) & 15) == 0 && blocks < 65536) {
    const dim3 few((bw + 7) / 8, blocks, (n_tokens + AF_GF_TM - 1) / AF_GF_TM);
    AF_DISPATCH_DTYPE(w_dtype, TW,
                      af_launch(gate_rows_few_kernel<TW>, few, dim3(256), (size_t)AF_GF_TM * bw * sizeof(float), stream,
                                decay, input, u, (const TW*)wa, (const TW*)wi, ba, bi, rate, n_tokens, width, bw));
    AF_CHECK_LAUNCH("af_gate_rows");
  }
  const dim3 grid((n_tokens + AF_GR_TM - 1) / AF_GR_TM, blocks, (bw + AF_GR_TN - 1) / AF_GR_TN);
  AF_REQUIRE(grid.y < 65536 && grid.z < 65536, "af_gate_rows: too many blocks of channels");
  AF_DISPATCH_DTYPE(w_dtype, TW,
                    af_launch(gate_rows_kernel<TW>, grid, dim3(256), 0, stream, decay, input, u, (const TW*)wa,
                              (const TW*)wi, ba, bi, rate, n_tokens, width, bw));
  AF_CHECK_LAUNCH("af_gate_rows");
}

// ---------------------------------------------------------------- the recurrence

__device__ __forceinline__ float gelu_tanh_f32(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// A block owns 32 channels of a sequence (a lane each) and walks its tokens 128 at a time: warp w takes 16 tokens
// in a row and composes their maps S -> S - d S + b (d = 1 - a; two such maps compose to d = d1 + d2 - d1 d2),
// the warps exchange the pairs, each warp composes the pairs of the
// warps before it onto the state carried so far and then walks its tokens from the state that really enters them.
#define AF_DS_WARPS 16      // at most; a step of single tokens runs with one
#define AF_DS_RUN 16
template <typename TY>
__global__ void __launch_bounds__(AF_DS_WARPS * 32)
decay_scan_kernel(TY* __restrict__ out, const float* __restrict__ decay, const float* __restrict__ input,
                  const float* __restrict__ proj, long long ld, int off_y, int off_x, const float* __restrict__ by,
                  const float* __restrict__ bx, float* __restrict__ state, const int* __restrict__ seq_starts,
                  const int* __restrict__ slots, int width, int taps) {
  pdl_launch_dependents();
  __shared__ float comp[AF_DS_WARPS][32][2];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  const int b = blockIdx.y;
  const bool on = c < width;
  const int first = seq_starts[b], last = seq_starts[b + 1];
  const int slot = slots[b];
  const float yb = on ? by[c] : 0.f;
  pdl_wait();
  decay = pdl_fresh(decay);
  input = pdl_fresh(input);
  proj = pdl_fresh(proj);
  if (slot < 0) {
    if (on)
      for (int t = first + w; t < last; t += nw) out[(size_t)t * width + c] = from_f32<TY>(0.f);
    return;
  }
  float* srow = state + (size_t)slot * taps * width;
  float carry = on ? srow[c] : 0.f;
  for (int base = first; base < last; base += nw * AF_DS_RUN) {
    const int t0 = base + w * AF_DS_RUN;
    const int n = max(0, min(AF_DS_RUN, last - t0));
    float a[AF_DS_RUN], v[AF_DS_RUN], g[AF_DS_RUN];
#pragma unroll
    for (int e = 0; e < AF_DS_RUN; ++e) {
      const bool in = on && e < n;
      const size_t at = (size_t)(t0 + e) * width + c;
      a[e] = in ? decay[at] : 0.f;                 // 1 - a of the token
      v[e] = in ? input[at] : 0.f;
      g[e] = in ? proj[(size_t)(t0 + e) * ld + off_y + c] : 0.f;
    }
    float A = 0.f, B = 0.f;                        // the stretch's map: S -> S - A S + B
#pragma unroll
    for (int e = 0; e < AF_DS_RUN; ++e) {
      if (e < n) {
        A = fmaf(-A, a[e], A + a[e]);
        B = fmaf(-a[e], B, B) + v[e];
      }
    }
    comp[w][lane][0] = A;
    comp[w][lane][1] = B;
    __syncthreads();
    float S = carry, full = carry;
    for (int x = 0; x < nw; ++x) {
      if (x == w) S = full;
      full = fmaf(-comp[x][lane][0], full, full) + comp[x][lane][1];
    }
    carry = full;
#pragma unroll
    for (int e = 0; e < AF_DS_RUN; ++e) {
      if (e < n) {
        S = fmaf(-a[e], S, S) + v[e];
        if (on) out[(size_t)(t0 + e) * width + c] = from_f32<TY>(S * gelu_tanh_f32(g[e] + yb));
      }
    }
    __syncthreads();
  }
  if (!on || w != 0) return;
  srow[c] = carry;
  // the convolution's last taps - 1 inputs: those of the step's last tokens, and before them what the state held
  const int n_new = last - first;
  const float xb = bx[c];
  for (int j = 1; j < taps; ++j) {                      // ascending: row j only takes from rows >= j
    const int src = n_new - (taps - j);                 // index among the step's tokens (negative: before the step)
    float v;
    if (src >= 0) v = proj[(size_t)(first + src) * ld + off_x + c] + xb;
    else v = srow[(size_t)(taps + src) * width + c];
    srow[(size_t)j * width + c] = v;
  }
}

AF_EXPORT int af_decay_scan(void* out, int out_dtype, const float* decay, const float* input, const float* proj,
                            long long ld, int off_y, int off_x, const float* by, const float* bx, float* state,
                            const int* seq_starts, const int* slots, int n_seqs, int n_tokens, int width, int taps,
                            cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  AF_REQUIRE(n_seqs > 0 && n_seqs < 65536 && n_tokens >= 0 && width > 0 && taps >= 1, "af_decay_scan: bad sizes");
  // warps by the tokens a sequence is likely to have in this step (any number is correct): one for single tokens,
  // up to AF_DS_WARPS for a prompt
  const int most = n_tokens - (n_seqs - 1);
  int warps = 1;
  while (warps < AF_DS_WARPS && warps * AF_DS_RUN < most) warps *= 2;
  AF_DISPATCH_DTYPE(out_dtype, TY,
                    af_launch(decay_scan_kernel<TY>, dim3((width + 31) / 32, n_seqs), dim3(warps * 32), 0, stream,
                              (TY*)out, decay, input, proj, ld, off_y, off_x, by, bx, state, seq_starts, slots, width,
                              taps));
  AF_CHECK_LAUNCH("af_decay_scan");
}
