// Mixers that carry a state of fixed size from token to token instead of keys
// and values: matrix-valued states per head (linear attention with a decay per
// head; the generalized delta rule with a decay per key channel and a removal
// term) and vector-valued states (a gated recurrence whose gates read only the
// current token).  The state and everything that enters the recurrence is
// 32-bit in both precisions; the kernels read the projections as 32-bit rows.
//
// A state of one sequence, run and head is stored [value column][key channel]:
// the key channels of a column lie together, so that the lanes that share a
// column read and write whole 16-byte pieces.
#include "common.cuh"

// ---------------------------------------------------------------- what enters the delta rule

// From the packed projection row of a token: per head and key channel c
//   unit key   u = k / sqrt(sum_c k^2 + key_eps)
//   decay      w = exp(-decay_scale * sigmoid(w2 . tanh(w1 row) + w0))
//   removal    au = sigmoid(a + a_bias) * u
// written as float rows [token][3][heads * dk] (w, u, au).  One block per (token, head), a thread per key
// channel; `w2t` is the second low-rank matrix transposed, [rank][heads * dk], so that the threads of a
// block read it side by side.
__global__ void __launch_bounds__(256)
delta_prep_kernel(float* __restrict__ out, const float* __restrict__ proj, long long ld, int off_k, int off_a,
                  int off_w1, const float* __restrict__ a_bias, const float* __restrict__ w0,
                  const float* __restrict__ w2t, int rank, int heads, int dk, float decay_scale, float key_eps) {
  pdl_launch_dependents();
  extern __shared__ float low[];                // tanh of the low-rank row
  __shared__ float scratch[33];
  const int t = blockIdx.x, h = blockIdx.y;
  const int n = heads * dk;
  // (weights before the wait for the projection)
  float bias_a[4], bias_w[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int c = threadIdx.x + e * blockDim.x;
    bias_a[e] = c < dk ? a_bias[h * dk + c] : 0.f;
    bias_w[e] = c < dk ? w0[h * dk + c] : 0.f;
  }
  pdl_wait();
  const float* row = proj + (size_t)t * ld;
  for (int l = threadIdx.x; l < rank; l += blockDim.x) low[l] = tanhf(row[off_w1 + l]);
  float kv[4], av[4], ss = 0.f;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int c = threadIdx.x + e * blockDim.x;
    kv[e] = c < dk ? row[off_k + h * dk + c] : 0.f;
    av[e] = c < dk ? row[off_a + h * dk + c] : 0.f;
    ss += kv[e] * kv[e];
  }
  ss = block_sum(ss, scratch);                  // (its barriers also publish `low`)
  const float nrm = sqrtf(ss + key_eps);
  float* o = out + (size_t)t * 3 * n;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int c = threadIdx.x + e * blockDim.x;
    if (c >= dk) continue;
    const int i = h * dk + c;
    float z = bias_w[e];
    for (int l = 0; l < rank; ++l) z += low[l] * w2t[(size_t)l * n + i];
    const float sig = 1.f / (1.f + expf(-z));
    const float u = kv[e] / nrm;
    const float a = 1.f / (1.f + expf(-(av[e] + bias_a[e])));
    o[i] = expf(-decay_scale * sig);
    o[n + i] = u;
    o[2 * n + i] = a * u;
  }
}

AF_EXPORT int af_delta_prep(float* out, const float* proj, long long ld, int off_k, int off_a, int off_w1,
                            const float* a_bias, const float* w0, const float* w2t, int rank, int n_tokens, int heads,
                            int dk, float decay_scale, float key_eps, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && heads > 0 && heads < 65536 && dk > 0 && dk <= 1024 && rank > 0 && rank <= 8192,
             "af_delta_prep: bad sizes (key size up to 1024, rank up to 8192)");
  const int threads = dk <= 32 ? 32 : dk <= 64 ? 64 : dk <= 128 ? 128 : 256;
  af_launch(delta_prep_kernel, dim3(n_tokens, heads), dim3(threads), (size_t)rank * sizeof(float), stream, out, proj, ld,
            off_k, off_a, off_w1, a_bias, w0, w2t, rank, heads, dk, decay_scale, key_eps);
  AF_CHECK_LAUNCH("af_delta_prep");
}

// ---------------------------------------------------------------- the scan over a matrix state

enum AfScanMode { AF_SCAN_DECAY = 0, AF_SCAN_DELTA = 1, AF_SCAN_CHANNEL = 3 };
// (inside the library: the decay recurrence whose r, k and v pass through SiLU as they are read; a kernel of
// its own, so that the others carry no exponentials)
#define AF_SCAN_DECAY_SILU 2

// The vectors of a token and head that the scan reads (float rows; `*_ts` is the distance between
// tokens in elements; head h's piece starts h * dk (h * dv for v) behind the pointer):
//   DECAY:  S <- decay[h] S + k v^T                          o = S^T q     (q = `r`)
//   DELTA:  S <- diag(w) S - au (u^T S) + k v^T              o = S^T r     (decay and removal act on the S before the token)
//   CHANNEL: S <- diag(w) S + k v^T                          o = S^T q     (a decay per key channel and token, no removal)
// With `silu` the r, k and v values go through x / (1 + exp(-x)) as they are read.
struct AfScanArgs {
  const float *r, *k, *v, *w, *u, *au;
  long long r_ts, k_ts, v_ts, w_ts, u_ts, au_ts;
  const float* decay;          // [heads] (DECAY)
  float* state;                // [slots][heads][dv][dk]
  float* out;                  // [tokens][heads * dv]
  long long out_ts;
  const int* seq_starts;       // [sequences + 1] first row of each sequence of the step
  const int* slots;            // [sequences] state slot, -1: a padding row (nothing read or written but zeros out)
  int heads, dk, dv;
  int lanes;                   // P: lanes that share a value column (a power of two); lane p holds key channels p R .. p R + R - 1
  int cols;                    // value columns of a block
  int chunk;                   // tokens staged in shared memory at a time
  int silu;
};

// Floats of padding behind a lane's run of R staged key channels: the 16-byte reads of a quarter warp (eight
// lanes, a run apart) then fall into different banks.  Runs of four floats lie side by side as they are.
#define AF_SCAN_PAD(R) ((R) == 4 ? 0 : 4)
#define AF_SCAN_PREFETCH 24    // values a thread holds in registers for the chunk after the current one
#define AF_SCAN_VEC_ITEMS 2    // the same in 16-byte pieces, per vector, where the sizes allow whole pieces

// Sum over the P lanes that share a column (P a power of two up to 32; the lanes of a group are neighbours).
__device__ __forceinline__ float lanes_sum(float v, int P) {
  if (P > 1) v += __shfl_xor_sync(0xffffffffu, v, 1);
  if (P > 2) v += __shfl_xor_sync(0xffffffffu, v, 2);
  if (P > 4) v += __shfl_xor_sync(0xffffffffu, v, 4);
  if (P > 8) v += __shfl_xor_sync(0xffffffffu, v, 8);
  if (P > 16) v += __shfl_xor_sync(0xffffffffu, v, 16);
  return v;
}

// One block per (column tile, head, sequence); thread = (column, lane of the column).  The block walks
// the sequence's tokens in chunks: while it scans a chunk out of shared memory, the next chunk's vectors
// are on their way into registers.  Key channel c lives at (c / R) (R + pad) + c % R of a staged vector (four
// floats of padding per lane's run keep the 16-byte reads of a quarter warp in different banks).
template <int R, int MODE, bool VEC>
__global__ void __launch_bounds__(256)
state_scan_kernel(AfScanArgs a) {
  pdl_launch_dependents();
  constexpr bool SILU = MODE == AF_SCAN_DECAY_SILU;
  extern __shared__ __align__(16) float smem[];
  const int P = a.lanes, CT = a.cols, CH = a.chunk, dk = a.dk, dv = a.dv;
  const int NV = MODE == AF_SCAN_DELTA ? 5 : MODE == AF_SCAN_CHANNEL ? 3 : 2;   // staged key-sized vectors: r, k (, w (, u, au))
  const int dkp = P * (R + AF_SCAN_PAD(R));
  const int tok_floats = NV * dkp + CT;                     // a token's staged floats: the vectors, then its v tile
  const int buf_floats = CH * tok_floats;
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int part = tid % P, col = tid / P;
  const int h = blockIdx.y, b = blockIdx.z;
  const int j0 = blockIdx.x * CT, j = j0 + col;
  const bool col_on = j < dv;
  // a token's values in the order they are fetched: NV key vectors of dk, then CT values of v
  const int tok_vals = NV * dk + CT;
  const int first = a.seq_starts[b], last = a.seq_starts[b + 1];
  const int slot = a.slots[b];
  pdl_wait();
  if (slot < 0) {
    for (int t = first + tid / CT; t < last; t += nthr / CT)
      if (j0 + tid % CT < dv) a.out[(size_t)t * a.out_ts + h * dv + j0 + tid % CT] = 0.f;
    return;
  }
  // the state's piece of this thread (16-byte pieces where the key size allows)
  float S[R];
  float* st = a.state + (((size_t)slot * a.heads + h) * dv + (col_on ? j : 0)) * dk + part * R;
  const bool vec = (dk & 3) == 0;
  if (vec) {
#pragma unroll
    for (int i = 0; i < R; i += 4) {
      float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
      if (col_on && part * R + i < dk) q = *reinterpret_cast<const float4*>(st + i);
      S[i] = q.x, S[i + 1] = q.y, S[i + 2] = q.z, S[i + 3] = q.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < R; ++i) S[i] = (col_on && part * R + i < dk) ? st[i] : 0.f;
  }
  const float dec = (MODE == AF_SCAN_DECAY || MODE == AF_SCAN_DECAY_SILU) ? a.decay[h] : 0.f;
  auto keep_state = [&]() {
    if (!col_on) return;
    if (vec) {
#pragma unroll
      for (int i = 0; i < R; i += 4)
        if (part * R + i < dk) *reinterpret_cast<float4*>(st + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < R; ++i)
        if (part * R + i < dk) st[i] = S[i];
    }
  };

  for (int i = tid; i < 2 * buf_floats; i += nthr) smem[i] = 0.f;        // (the padding stays zero for good)

  // The loads of a chunk are all issued before any of their values is used (what is done to a value, the
  // activation, is done when it is staged).  Which tokens and channels a thread fetches does not change from
  // chunk to chunk: the places are worked out once.
  constexpr int FE = VEC ? AF_SCAN_VEC_ITEMS : AF_SCAN_PREFETCH;   // key-vector items a thread fetches (per vector if VEC)
  constexpr int FV = VEC ? AF_SCAN_VEC_ITEMS : 1;                  // value-tile items
  float4 pq[VEC ? 5 : 1][VEC ? FE : 1], pvq[FV];
  float pf[VEC ? 1 : AF_SCAN_PREFETCH];
  int ftt[VEC ? FE : 1], fgo[VEC ? FE : 1], fso[VEC ? FE : 1], vtt[FV], vgo[FV], vso[FV];
  if constexpr (VEC) {
    const int dkq = dk >> 2, ctq = CT >> 2;
#pragma unroll
    for (int e = 0; e < FE; ++e) {
      const int idx = tid + e * nthr;
      const int tt = idx / dkq, c = (idx - tt * dkq) * 4;
      ftt[e] = idx < CH * dkq ? tt : CH;                     // (CH: never among a chunk's tokens)
      fgo[e] = h * dk + c;
      fso[e] = tt * tok_floats + (c / R) * (R + AF_SCAN_PAD(R)) + c % R;
    }
#pragma unroll
    for (int e = 0; e < FV; ++e) {
      const int idx = tid + e * nthr;
      const int tt = idx / ctq, x = (idx - tt * ctq) * 4;
      vtt[e] = (idx < CH * ctq && j0 + x < dv) ? tt : CH;
      vgo[e] = h * dv + j0 + x;
      vso[e] = tt * tok_floats + NV * dkp + x;
    }
  }
  auto act4 = [&](float4 q) {
    q.x = q.x / (1.f + expf(-q.x)), q.y = q.y / (1.f + expf(-q.y));
    q.z = q.z / (1.f + expf(-q.z)), q.w = q.w / (1.f + expf(-q.w));
    return q;
  };
  auto fetch = [&](int t0, int n) {                          // tokens t0 .. t0 + n - 1 into registers
    if constexpr (VEC) {
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        const float* p = v == 0 ? a.r : v == 1 ? a.k : v == 2 ? a.w : v == 3 ? a.u : a.au;
        const long long ts = v == 0 ? a.r_ts : v == 1 ? a.k_ts : v == 2 ? a.w_ts : v == 3 ? a.u_ts : a.au_ts;
#pragma unroll
        for (int e = 0; e < FE; ++e)
          if (ftt[e] < n) pq[v][e] = *reinterpret_cast<const float4*>(p + (size_t)(t0 + ftt[e]) * ts + fgo[e]);
      }
#pragma unroll
      for (int e = 0; e < FV; ++e)
        if (vtt[e] < n) pvq[e] = *reinterpret_cast<const float4*>(a.v + (size_t)(t0 + vtt[e]) * a.v_ts + vgo[e]);
    } else {
#pragma unroll
      for (int e = 0; e < AF_SCAN_PREFETCH; ++e) {
        const int idx = tid + e * nthr;
        float val = 0.f;
        if (idx < n * tok_vals) {
          const int tt = idx / tok_vals, x = idx - tt * tok_vals;
          const size_t t = (size_t)(t0 + tt);
          if (x < NV * dk) {
            const int vec = x / dk, c = x - vec * dk;
            const float* p = vec == 0 ? a.r + t * a.r_ts : vec == 1 ? a.k + t * a.k_ts
                           : vec == 2 ? a.w + t * a.w_ts : vec == 3 ? a.u + t * a.u_ts : a.au + t * a.au_ts;
            val = p[h * dk + c];
          } else {
            const int jj = j0 + x - NV * dk;
            if (jj < dv) val = a.v[t * a.v_ts + h * dv + jj];
          }
        }
        pf[e] = val;
      }
    }
  };
  auto stage = [&](float* buf, int n) {                      // registers into a shared-memory buffer
    if constexpr (VEC) {
#pragma unroll
      for (int v = 0; v < NV; ++v)
#pragma unroll
        for (int e = 0; e < FE; ++e)
          if (ftt[e] < n)
            *reinterpret_cast<float4*>(buf + fso[e] + v * dkp) = (SILU && v < 2) ? act4(pq[v][e]) : pq[v][e];
#pragma unroll
      for (int e = 0; e < FV; ++e)
        if (vtt[e] < n) *reinterpret_cast<float4*>(buf + vso[e]) = SILU ? act4(pvq[e]) : pvq[e];
    } else {
#pragma unroll
      for (int e = 0; e < AF_SCAN_PREFETCH; ++e) {
        const int idx = tid + e * nthr;
        if (idx < n * tok_vals) {
          const int tt = idx / tok_vals, x = idx - tt * tok_vals;
          int at;
          bool act = SILU;
          if (x < NV * dk) {
            const int vec = x / dk, c = x - vec * dk;
            at = vec * dkp + (c / R) * (R + AF_SCAN_PAD(R)) + c % R;
            act = act && vec < 2;
          } else {
            at = NV * dkp + x - NV * dk;
          }
          buf[tt * tok_floats + at] = act ? pf[e] / (1.f + expf(-pf[e])) : pf[e];
        }
      }
    }
  };

  int t0 = first;
  int n = min(CH, last - t0);
  fetch(t0, n);
  __syncthreads();                                           // (the zeroing is done)
  int which = 0;
  while (t0 < last) {
    float* buf = smem + which * buf_floats;
    stage(buf, n);
    __syncthreads();
    const int t1 = t0 + n;
    const int n1 = min(CH, last - t1);
    if (n1 > 0) fetch(t1, n1);                               // under the scan of this chunk
#pragma unroll 2
    for (int tt = 0; tt < n; ++tt) {
      const float* tk = buf + tt * tok_floats + part * (R + AF_SCAN_PAD(R));
      const float vj = buf[tt * tok_floats + NV * dkp + col];
      float rv[R], kv[R];
#pragma unroll
      for (int i = 0; i < R; i += 4) {
        *reinterpret_cast<float4*>(rv + i) = *reinterpret_cast<const float4*>(tk + i);
        *reinterpret_cast<float4*>(kv + i) = *reinterpret_cast<const float4*>(tk + dkp + i);
      }
      if (MODE == AF_SCAN_DELTA) {
        float wv[R], uv[R], av[R];
#pragma unroll
        for (int i = 0; i < R; i += 4) {
          *reinterpret_cast<float4*>(wv + i) = *reinterpret_cast<const float4*>(tk + 2 * dkp + i);
          *reinterpret_cast<float4*>(uv + i) = *reinterpret_cast<const float4*>(tk + 3 * dkp + i);
          *reinterpret_cast<float4*>(av + i) = *reinterpret_cast<const float4*>(tk + 4 * dkp + i);
        }
        float d0 = 0.f, d1 = 0.f;
#pragma unroll
        for (int i = 0; i < R; i += 2) {
          d0 += uv[i] * S[i];
          d1 += uv[i + 1] * S[i + 1];
        }
        const float dot = lanes_sum(d0 + d1, P);
#pragma unroll
        for (int i = 0; i < R; ++i) S[i] = wv[i] * S[i] - av[i] * dot + kv[i] * vj;
      } else if (MODE == AF_SCAN_CHANNEL) {
        float wv[R];
#pragma unroll
        for (int i = 0; i < R; i += 4)
          *reinterpret_cast<float4*>(wv + i) = *reinterpret_cast<const float4*>(tk + 2 * dkp + i);
#pragma unroll
        for (int i = 0; i < R; ++i) S[i] = wv[i] * S[i] + kv[i] * vj;
      } else {
#pragma unroll
        for (int i = 0; i < R; ++i) S[i] = dec * S[i] + kv[i] * vj;
      }
      float o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int i = 0; i < R; i += 2) {
        o0 += rv[i] * S[i];
        o1 += rv[i + 1] * S[i + 1];
      }
      const float o = lanes_sum(o0 + o1, P);
      if (part == 0 && col_on) a.out[(size_t)(t0 + tt) * a.out_ts + h * dv + j] = o;
    }
    t0 = t1;
    n = n1;
    which ^= 1;
  }
  keep_state();
}

// A step in which every sequence brings one token (a decode step): one block per (column tile, head,
// sequence) as above, but nothing is staged: the token's vectors go from memory to the lanes' registers, the
// state's tile is read, updated and written back.  `vec`: whole 16-byte pieces.
template <int R, int MODE>
__global__ void __launch_bounds__(256)
state_step_kernel(AfScanArgs a, int vec) {
  pdl_launch_dependents();
  constexpr bool SILU = MODE == AF_SCAN_DECAY_SILU;
  const int P = a.lanes, CT = a.cols, dk = a.dk, dv = a.dv;
  const int tid = threadIdx.x;
  const int part = tid % P, col = tid / P;
  const int h = blockIdx.y, b = blockIdx.z;
  const int j = blockIdx.x * CT + col;
  const bool col_on = j < dv;
  const int slot = a.slots[b];
  const size_t t = (size_t)a.seq_starts[b];
  const int c0 = part * R;
  if (slot < 0) {
    pdl_wait();
    if (part == 0 && col_on) a.out[t * a.out_ts + h * dv + j] = 0.f;
    return;
  }
  // the state is what the step before left: it does not wait for the kernel in front
  float S[R];
  float* st = a.state + (((size_t)slot * a.heads + h) * dv + (col_on ? j : 0)) * dk + c0;
  if (vec) {
#pragma unroll
    for (int i = 0; i < R; i += 4) {
      float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
      if (col_on && c0 + i < dk) q = *reinterpret_cast<const float4*>(st + i);
      S[i] = q.x, S[i + 1] = q.y, S[i + 2] = q.z, S[i + 3] = q.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < R; ++i) S[i] = (col_on && c0 + i < dk) ? st[i] : 0.f;
  }
  const float dec = (MODE == AF_SCAN_DECAY || MODE == AF_SCAN_DECAY_SILU) ? a.decay[h] : 0.f;
  pdl_wait();
  auto piece = [&](const float* p, float* dst, bool act) {
    p += h * dk + c0;
    if (vec) {
#pragma unroll
      for (int i = 0; i < R; i += 4) {
        float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c0 + i < dk) q = *reinterpret_cast<const float4*>(p + i);
        dst[i] = q.x, dst[i + 1] = q.y, dst[i + 2] = q.z, dst[i + 3] = q.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < R; ++i) dst[i] = c0 + i < dk ? p[i] : 0.f;
    }
    if (act) {
#pragma unroll
      for (int i = 0; i < R; ++i) dst[i] = dst[i] / (1.f + expf(-dst[i]));
    }
  };
  float rv[R], kv[R];
  piece(a.r + t * a.r_ts, rv, SILU);
  piece(a.k + t * a.k_ts, kv, SILU);
  float vj = col_on ? a.v[t * a.v_ts + h * dv + j] : 0.f;
  if (SILU) vj = vj / (1.f + expf(-vj));
  if (MODE == AF_SCAN_DELTA) {
    float wv[R], uv[R], av[R];
    piece(a.w + t * a.w_ts, wv, false);
    piece(a.u + t * a.u_ts, uv, false);
    piece(a.au + t * a.au_ts, av, false);
    float d0 = 0.f, d1 = 0.f;
#pragma unroll
    for (int i = 0; i < R; i += 2) d0 += uv[i] * S[i], d1 += uv[i + 1] * S[i + 1];
    const float dot = lanes_sum(d0 + d1, P);
#pragma unroll
    for (int i = 0; i < R; ++i) S[i] = wv[i] * S[i] - av[i] * dot + kv[i] * vj;
  } else if (MODE == AF_SCAN_CHANNEL) {
    float wv[R];
    piece(a.w + t * a.w_ts, wv, false);
#pragma unroll
    for (int i = 0; i < R; ++i) S[i] = wv[i] * S[i] + kv[i] * vj;
  } else {
#pragma unroll
    for (int i = 0; i < R; ++i) S[i] = dec * S[i] + kv[i] * vj;
  }
  float o0 = 0.f, o1 = 0.f;
#pragma unroll
  for (int i = 0; i < R; i += 2) o0 += rv[i] * S[i], o1 += rv[i + 1] * S[i + 1];
  const float o = lanes_sum(o0 + o1, P);
  if (part == 0 && col_on) a.out[t * a.out_ts + h * dv + j] = o;
  if (!col_on) return;
  if (vec) {
#pragma unroll
    for (int i = 0; i < R; i += 4)
      if (c0 + i < dk) *reinterpret_cast<float4*>(st + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
  } else {
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (c0 + i < dk) st[i] = S[i];
  }
}

template <int R>
static int launch_step(const AfScanArgs& a, int mode, int vec, dim3 grid, int threads, cudaStream_t stream) {
  if (mode == AF_SCAN_DELTA) af_launch(state_step_kernel<R, AF_SCAN_DELTA>, grid, dim3(threads), 0, stream, a, vec);
  else if (mode == AF_SCAN_CHANNEL) af_launch(state_step_kernel<R, AF_SCAN_CHANNEL>, grid, dim3(threads), 0, stream, a, vec);
  else if (a.silu) af_launch(state_step_kernel<R, AF_SCAN_DECAY_SILU>, grid, dim3(threads), 0, stream, a, vec);
  else af_launch(state_step_kernel<R, AF_SCAN_DECAY>, grid, dim3(threads), 0, stream, a, vec);
  AF_CHECK_LAUNCH("af_state_scan");
}

template <int R, bool VEC>
static int launch_scan(const AfScanArgs& a, int mode, dim3 grid, int threads, size_t smem, cudaStream_t stream) {
  static bool raised[4][AF_MAX_DEVICES];
  auto k0 = state_scan_kernel<R, AF_SCAN_DECAY, VEC>;
  auto k1 = state_scan_kernel<R, AF_SCAN_DELTA, VEC>;
  auto k2 = state_scan_kernel<R, AF_SCAN_DECAY_SILU, VEC>;
  auto k3 = state_scan_kernel<R, AF_SCAN_CHANNEL, VEC>;
  const int which = mode == AF_SCAN_DELTA ? 1 : mode == AF_SCAN_CHANNEL ? 3 : (a.silu ? 2 : 0);
  if (smem > 48 * 1024) {
    const int dev = af_current_device();
    if (dev < 0) return -1;
    if (af_first_on_device(raised[which], dev)) {
      cudaError_t e = cudaFuncSetAttribute(which == 1 ? k1 : which == 2 ? k2 : which == 3 ? k3 : k0, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           96 * 1024);
      if (e != cudaSuccess) return af_fail((int)e, "af_state_scan: %s", cudaGetErrorString(e));
    }
  }
  if (which == 1) af_launch(k1, grid, dim3(threads), smem, stream, a);
  else if (which == 2) af_launch(k2, grid, dim3(threads), smem, stream, a);
  else if (which == 3) af_launch(k3, grid, dim3(threads), smem, stream, a);
  else af_launch(k0, grid, dim3(threads), smem, stream, a);
  AF_CHECK_LAUNCH("af_state_scan");
}

// The cut of a scan: R key channels a lane, P lanes a column, CT columns a block, CH tokens a chunk.
// `vec`: the vectors are fetched in 16-byte pieces.  `want_blocks`: the device's SMs (what "a small step" is measured by).
static void scan_cut(int mode, int dk, int dv, bool vec, long long units, int want_blocks, int* R, int* P, int* CT,
                     int* CH) {
  // A token costs a lane a chain of instructions as long as its share of the key channels: while the whole
  // step has no more threads than two blocks an SM hold (a prompt or two: all blocks run at once), a column gets up to sixteen lanes;
  // with more work than that, eight lanes at most (fewer shuffles and less staging a state element).
  int r = 4, p = 1;
  for (;; r *= 2) {
    p = 1;
    while (p * r < dk && p < 32) p *= 2;
    if (r == 32 || (p * r >= dk && (p <= 8 || (p <= 16 && units * dv * p <= (long long)want_blocks * 256)))) break;
  }
  // 256 threads a block (512 measured the same or slower): every block of a head stages the head's vectors for itself, so wide tiles of columns
  // (few blocks a head, many warps a block) cost less than narrow ones, also where that leaves SMs without a block
  int ct = 256 / p;
  while (ct > 4 && ct / 2 >= dv && (ct / 2) * p >= 32) ct /= 2;   // (no wider than the state's columns need; whole warps)
  const int nv = mode == AF_SCAN_DELTA ? 5 : mode == AF_SCAN_CHANNEL ? 3 : 2;
  const int tok_vals = nv * dk + ct, tok_floats = nv * p * (r + AF_SCAN_PAD(r)) + ct;
  const int threads = ct * p;
  int ch = 16;
  while (ch > 1 && 2 * ch * tok_floats * 4 > 96 * 1024) ch /= 2;
  if (vec) {
    while (ch > 1 && (ch * (dk / 4) > AF_SCAN_VEC_ITEMS * threads || ch * (ct / 4) > AF_SCAN_VEC_ITEMS * threads)) ch /= 2;
  } else {
    while (ch > 1 && ch * tok_vals > AF_SCAN_PREFETCH * threads) ch /= 2;
  }
  *R = r, *P = p, *CT = ct, *CH = ch;
}

AF_EXPORT int af_state_scan(int mode, const float* r, long long r_ts, const float* k, long long k_ts, const float* v,
                            long long v_ts, const float* w, long long w_ts, const float* u, long long u_ts,
                            const float* au, long long au_ts, const float* decay, float* state, float* out,
                            long long out_ts, const int* seq_starts, const int* slots, int n_seqs, int n_tokens, int heads,
                            int dk, int dv, int silu, cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  AF_REQUIRE(mode == AF_SCAN_DECAY || mode == AF_SCAN_DELTA || mode == AF_SCAN_CHANNEL, "af_state_scan: mode %d", mode);
  AF_REQUIRE(!(mode != AF_SCAN_DECAY && silu), "af_state_scan: only the plain decay takes its vectors through SiLU");
  AF_REQUIRE(n_seqs > 0 && heads > 0 && dk > 0 && dv > 0 && dk <= 1024, "af_state_scan: bad sizes (key size up to 1024)");
  AF_REQUIRE(n_seqs < 65536 && heads < 65536, "af_state_scan: too many sequences or heads for one grid");
  AfScanArgs a;
  a.r = r, a.k = k, a.v = v, a.w = w, a.u = u, a.au = au;
  a.r_ts = r_ts, a.k_ts = k_ts, a.v_ts = v_ts, a.w_ts = w_ts, a.u_ts = u_ts, a.au_ts = au_ts;
  a.decay = decay, a.state = state, a.out = out, a.out_ts = out_ts, a.seq_starts = seq_starts, a.slots = slots;
  a.heads = heads, a.dk = dk, a.dv = dv, a.silu = silu;
  // whole 16-byte pieces: sizes and strides in multiples of four floats, bases on 16 bytes
  bool vec = dk % 4 == 0 && dv % 4 == 0 && ((r_ts | k_ts | v_ts) & 3) == 0 &&
             (((uintptr_t)r | (uintptr_t)k | (uintptr_t)v) & 15) == 0;
  if (mode == AF_SCAN_CHANNEL) vec = vec && (w_ts & 3) == 0 && ((uintptr_t)w & 15) == 0;
  if (mode == AF_SCAN_DELTA)
    vec = vec && ((w_ts | u_ts | au_ts) & 3) == 0 && (((uintptr_t)w | (uintptr_t)u | (uintptr_t)au) & 15) == 0;
  const int sms = af_sm_count();
  if (sms <= 0) return -1;
  int R, P, CT, CH;
  scan_cut(mode, dk, dv, vec, (long long)heads * n_seqs, sms, &R, &P, &CT, &CH);
  AF_REQUIRE(P * R >= dk, "af_state_scan: key size %d does not fit %d lanes of %d", dk, P, R);
  const int nv = mode == AF_SCAN_DELTA ? 5 : mode == AF_SCAN_CHANNEL ? 3 : 2;
  if (vec)
    AF_REQUIRE(CH * (dk / 4) <= AF_SCAN_VEC_ITEMS * CT * P && CH * (CT / 4) <= AF_SCAN_VEC_ITEMS * CT * P,
               "af_state_scan: a token of %d values is too long to stage", nv * dk + CT);
  else
    AF_REQUIRE(CH * (nv * dk + CT) <= AF_SCAN_PREFETCH * CT * P, "af_state_scan: a token of %d values is too long to stage",
               nv * dk + CT);
  a.lanes = P, a.cols = CT, a.chunk = CH;
  if (n_tokens == n_seqs) {                                  // every sequence brings one token
    const dim3 grid((dv + CT - 1) / CT, heads, n_seqs);
    switch (R) {
      case 4: return launch_step<4>(a, mode, vec ? 1 : 0, grid, CT * P, stream);
      case 8: return launch_step<8>(a, mode, vec ? 1 : 0, grid, CT * P, stream);
      case 16: return launch_step<16>(a, mode, vec ? 1 : 0, grid, CT * P, stream);
      default: return launch_step<32>(a, mode, vec ? 1 : 0, grid, CT * P, stream);
    }
  }
  const size_t smem = (size_t)2 * CH * (nv * P * (R + AF_SCAN_PAD(R)) + CT) * sizeof(float);
  const dim3 grid((dv + CT - 1) / CT, heads, n_seqs);
  const int threads = CT * P;
  if (vec) {
    switch (R) {
      case 4: return launch_scan<4, true>(a, mode, grid, threads, smem, stream);
      case 8: return launch_scan<8, true>(a, mode, grid, threads, smem, stream);
      case 16: return launch_scan<16, true>(a, mode, grid, threads, smem, stream);
      default: return launch_scan<32, true>(a, mode, grid, threads, smem, stream);
    }
  }
  switch (R) {
    case 4: return launch_scan<4, false>(a, mode, grid, threads, smem, stream);
    case 8: return launch_scan<8, false>(a, mode, grid, threads, smem, stream);
    case 16: return launch_scan<16, false>(a, mode, grid, threads, smem, stream);
    default: return launch_scan<32, false>(a, mode, grid, threads, smem, stream);
  }
}

// ---------------------------------------------------------------- the output of a state mixer

// y[t][i] = o'[t][i] * rsqrt(mean over i's group of o'^2 + eps) * w[i] * sigmoid(gate[t][i]), o' = in_scale * o: a norm
// over groups of `group` values (a head, or the whole row) with a weight vector (no offset), times a gate (its sigmoid,
// or with gate_act 1 the gate times its sigmoid).  One block per token.
template <typename TY>
__global__ void __launch_bounds__(256)
gated_group_norm_kernel(TY* __restrict__ y, const float* __restrict__ o, const float* __restrict__ w,
                        const float* __restrict__ gate, long long gate_ts, int n, int group, float eps, int gate_act,
                        float in_scale) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  // the gate: its sigmoid, or (gate_act 1) the gate itself times its sigmoid
  auto gated = [&](float g) { const float sg = 1.f / (1.f + expf(-g)); return gate_act ? g * sg : sg; };
  const int t = blockIdx.x;
  const float* orow = o + (size_t)t * n;
  const float* grow = gate + (size_t)t * gate_ts;
  TY* yrow = y + (size_t)t * n;
  if (group == n) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss += (orow[i] * in_scale) * (orow[i] * in_scale);
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x)
      yrow[i] = from_f32<TY>(orow[i] * in_scale * inv * w[i] * gated(grow[i]));
    return;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  for (int g = warp; g < n / group; g += nwarp) {
    float ss = 0.f;
    for (int c = lane; c < group; c += 32) ss += (orow[g * group + c] * in_scale) * (orow[g * group + c] * in_scale);
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)group + eps);
    for (int c = lane; c < group; c += 32) {
      const int i = g * group + c;
      yrow[i] = from_f32<TY>(orow[i] * in_scale * inv * w[i] * gated(grow[i]));
    }
  }
}

AF_EXPORT int af_gated_group_norm(void* y, int y_dtype, const float* o, const float* w, const float* gate,
                                  long long gate_ts, int n_tokens, int n, int group, float eps, int gate_act,
                                  float in_scale, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && n > 0 && group > 0 && n % group == 0, "af_gated_group_norm: %d values in groups of %d", n, group);
  AF_DISPATCH_DTYPE(y_dtype, TY, af_launch(gated_group_norm_kernel<TY>, dim3(n_tokens), dim3(256), 0, stream, (TY*)y, o, w,
                                           gate, gate_ts, n, group, eps, gate_act, in_scale));
  AF_CHECK_LAUNCH("af_gated_group_norm");
}

// ---------------------------------------------------------------- a gated recurrence over a vector state

// Per channel: z = sigmoid(pz + bz), c = px + bx, candidate = c + 1/2 where c >= 0 and sigmoid(c) below,
// S <- (1 - z) S + z candidate, y = S * silu(pg).  pz, px, pg are sections of the packed projection row.
// A block owns 32 channels of a sequence (a lane each) and walks its tokens 128 at a time: warp w takes 16
// tokens in a row, works out what they do to any state that enters them (S_out = A S_in + B: the map of a
// token is affine, and so is their composition), the warps exchange these pairs, each warp composes the pairs
// of the warps before it onto the state carried so far, and then walks its 16 tokens once more from the state
// that really enters them.  The gates and candidates of the 16 tokens stay in registers between the passes.
#define AF_GS_WARPS 8
#define AF_GS_RUN 16
template <typename TY>
__global__ void __launch_bounds__(AF_GS_WARPS * 32)
gated_scan_kernel(TY* __restrict__ y, const float* __restrict__ proj, long long ld, int off_z, int off_x, int off_g,
                  const float* __restrict__ bz, const float* __restrict__ bx, float* __restrict__ state,
                  const int* __restrict__ seq_starts, const int* __restrict__ slots, int width) {
  pdl_launch_dependents();
  __shared__ float comp[AF_GS_WARPS][32][2];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  const int b = blockIdx.y;
  const bool on = c < width;
  const int first = seq_starts[b], last = seq_starts[b + 1];
  const int slot = slots[b];
  const float zb = on ? bz[c] : 0.f, xb = on ? bx[c] : 0.f;
  pdl_wait();
  if (slot < 0) {
    if (on)
      for (int t = first + w; t < last; t += AF_GS_WARPS) y[(size_t)t * width + c] = from_f32<TY>(0.f);
    return;
  }
  float carry = on ? state[(size_t)slot * width + c] : 0.f;
  for (int base = first; base < last; base += AF_GS_WARPS * AF_GS_RUN) {
    const int t0 = base + w * AF_GS_RUN;
    const int n = max(0, min(AF_GS_RUN, last - t0));
    float z[AF_GS_RUN], cd[AF_GS_RUN], g[AF_GS_RUN];
#pragma unroll
    for (int e = 0; e < AF_GS_RUN; ++e) {
      const bool in = on && e < n;
      const float* row = proj + (size_t)(t0 + e) * ld + c;
      z[e] = in ? row[off_z] : 0.f;
      cd[e] = in ? row[off_x] : 0.f;
      g[e] = in ? row[off_g] : 0.f;
    }
    float A = 1.f, B = 0.f;
#pragma unroll
    for (int e = 0; e < AF_GS_RUN; ++e) {
      if (e < n) {
        const float zz = 1.f / (1.f + expf(-(z[e] + zb)));
        const float u = cd[e] + xb;
        z[e] = zz;
        cd[e] = u >= 0.f ? u + 0.5f : 1.f / (1.f + expf(-u));
        A *= 1.f - zz;
        B = (1.f - zz) * B + zz * cd[e];
      }
    }
    comp[w][lane][0] = A;
    comp[w][lane][1] = B;
    __syncthreads();
    // the state that enters this warp's tokens, and the one that leaves the stretch (the same in every warp)
    float S = carry, full = carry;
    for (int v = 0; v < AF_GS_WARPS; ++v) {
      if (v == w) S = full;
      full = comp[v][lane][0] * full + comp[v][lane][1];
    }
    carry = full;
#pragma unroll
    for (int e = 0; e < AF_GS_RUN; ++e) {
      if (e < n) {
        S = (1.f - z[e]) * S + z[e] * cd[e];
        if (on) y[(size_t)(t0 + e) * width + c] = from_f32<TY>(S * (g[e] / (1.f + expf(-g[e]))));
      }
    }
    __syncthreads();
  }
  if (on && w == 0) state[(size_t)slot * width + c] = carry;
}

AF_EXPORT int af_gated_scan(void* y, int y_dtype, const float* proj, long long ld, int off_z, int off_x, int off_g,
                            const float* bz, const float* bx, float* state, const int* seq_starts, const int* slots,
                            int n_seqs, int width, cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  AF_REQUIRE(n_seqs > 0 && n_seqs < 65536 && width > 0, "af_gated_scan: bad sizes");
  AF_DISPATCH_DTYPE(y_dtype, TY, af_launch(gated_scan_kernel<TY>, dim3((width + 31) / 32, n_seqs), dim3(AF_GS_WARPS * 32), 0, stream,
                                           (TY*)y, proj, ld, off_z, off_x, off_g, bz, bx, state, seq_starts, slots, width));
  AF_CHECK_LAUNCH("af_gated_scan");
}

// ---------------------------------------------------------------- decays of gated linear attention

// alpha[t][c] = sigmoid(z)^(1 / tau), z = b[c] + sum_r w2t[r][c] * low[t][r], with low the `rank` columns of the packed
// float32 projection rows that begin at off_low (the first factor of a low-rank pair, applied with the other
// projections), w2t [rank, n] the second factor transposed.  Worked out as exp(log(sigmoid(z)) / tau) with
// log(sigmoid(z)) = min(z, 0) - log1p(exp(-|z|)): 32-bit throughout, no underflow of the sigmoid on the way.
// The sum over r is taken in AF_CD_SLICES runs of neighbouring r, each from zero, and the runs are added in order:
// both kernels below do exactly that, so a prompt and a decode step give the same bits.
//   many tokens: a block owns AF_CD_TOK tokens and 128 channels (a thread a channel); the tokens' low-rank rows lie
//                in shared memory and a value of w2t is read once for all of the block's tokens;
//   few tokens:  a block owns 32 channels, and a warp a run of r: every thread has only rank / AF_CD_SLICES loads
//                behind one another, and eight times as many warps stream the matrix.
#define AF_CD_TOK 16
#define AF_CD_SLICES 8

__device__ __forceinline__ float decay_of(float z, float inv_tau) {
  const float ls = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
  return expf(ls * inv_tau);
}

// z[.] += w2t[r][c] * low[r][.] for r in [r0, r1): the partial sum of one run, from zero
__device__ __forceinline__ void decay_run(float* p, const float* __restrict__ w2t, const float* low, int r0, int r1, int n,
                                          int c) {
#pragma unroll
  for (int tt = 0; tt < AF_CD_TOK; ++tt) p[tt] = 0.f;
#pragma unroll 8
  for (int r = r0; r < r1; ++r) {
    const float w = w2t[(size_t)r * n + c];
    const float4* lr = reinterpret_cast<const float4*>(low + r * AF_CD_TOK);
#pragma unroll
    for (int q = 0; q < AF_CD_TOK / 4; ++q) {
      const float4 l = lr[q];
      p[4 * q] = fmaf(w, l.x, p[4 * q]);
      p[4 * q + 1] = fmaf(w, l.y, p[4 * q + 1]);
      p[4 * q + 2] = fmaf(w, l.z, p[4 * q + 2]);
      p[4 * q + 3] = fmaf(w, l.w, p[4 * q + 3]);
    }
  }
}

__global__ void __launch_bounds__(128)
channel_decay_kernel(float* __restrict__ alpha, const float* __restrict__ proj, long long ld, int off_low,
                     const float* __restrict__ w2t, const float* __restrict__ bias, int rank, int n, int n_tokens,
                     float inv_tau) {
  pdl_launch_dependents();
  extern __shared__ __align__(16) float low[];                // [rank][AF_CD_TOK]
  const int t0 = blockIdx.y * AF_CD_TOK;
  const int c = blockIdx.x * 128 + threadIdx.x;
  const float b = c < n ? bias[c] : 0.f;
  pdl_wait();
  proj = pdl_fresh(proj);
  for (int i = threadIdx.x; i < rank * AF_CD_TOK; i += 128) {
    const int tt = i / rank, r = i - tt * rank;
    low[r * AF_CD_TOK + tt] = t0 + tt < n_tokens ? proj[(size_t)(t0 + tt) * ld + off_low + r] : 0.f;
  }
  __syncthreads();
  if (c >= n) return;
  const int per = (rank + AF_CD_SLICES - 1) / AF_CD_SLICES;
  float z[AF_CD_TOK];
#pragma unroll
  for (int tt = 0; tt < AF_CD_TOK; ++tt) z[tt] = 0.f;
  for (int s = 0; s < AF_CD_SLICES; ++s) {
    float p[AF_CD_TOK];
    decay_run(p, w2t, low, min(s * per, rank), min((s + 1) * per, rank), n, c);
#pragma unroll
    for (int tt = 0; tt < AF_CD_TOK; ++tt) z[tt] += p[tt];
  }
#pragma unroll
  for (int tt = 0; tt < AF_CD_TOK; ++tt) {
    if (t0 + tt >= n_tokens) break;
    alpha[(size_t)(t0 + tt) * n + c] = decay_of(z[tt] + b, inv_tau);
  }
}

// Up to AF_CD_TOK tokens: block = 32 channels x AF_CD_SLICES runs (warp s takes run s).
__global__ void __launch_bounds__(32 * AF_CD_SLICES)
channel_decay_few_kernel(float* __restrict__ alpha, const float* __restrict__ proj, long long ld, int off_low,
                         const float* __restrict__ w2t, const float* __restrict__ bias, int rank, int n, int n_tokens,
                         float inv_tau) {
  pdl_launch_dependents();
  extern __shared__ __align__(16) float low[];                // [rank][AF_CD_TOK], then the runs' sums [runs][tokens][32]
  float* sums = low + (size_t)rank * AF_CD_TOK;
  const int lane = threadIdx.x & 31, s = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  const float b = c < n ? bias[c] : 0.f;
  pdl_wait();
  proj = pdl_fresh(proj);
  for (int i = threadIdx.x; i < rank * AF_CD_TOK; i += blockDim.x) {
    const int tt = i / rank, r = i - tt * rank;
    low[r * AF_CD_TOK + tt] = tt < n_tokens ? proj[(size_t)tt * ld + off_low + r] : 0.f;
  }
  __syncthreads();
  const int per = (rank + AF_CD_SLICES - 1) / AF_CD_SLICES;
  float p[AF_CD_TOK];
  decay_run(p, w2t, low, min(s * per, rank), min((s + 1) * per, rank), n, c < n ? c : 0);
#pragma unroll
  for (int tt = 0; tt < AF_CD_TOK; ++tt) sums[(s * AF_CD_TOK + tt) * 32 + lane] = p[tt];
  __syncthreads();
  if (c >= n) return;
  for (int tt = s; tt < n_tokens; tt += AF_CD_SLICES) {       // warp s finishes tokens s, s + runs, ...
    float z = 0.f;
#pragma unroll
    for (int q = 0; q < AF_CD_SLICES; ++q) z += sums[(q * AF_CD_TOK + tt) * 32 + lane];
    alpha[(size_t)tt * n + c] = decay_of(z + b, inv_tau);
  }
}

AF_EXPORT int af_channel_decay(float* alpha, const float* proj, long long ld, int off_low, const float* w2t,
                               const float* bias, int rank, int n_tokens, int n, float tau, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  AF_REQUIRE(n_tokens > 0 && n > 0 && rank > 0 && rank <= 512 && tau > 0.f, "af_channel_decay: bad sizes (rank up to 512)");
  if (n_tokens <= AF_CD_TOK) {
    const size_t smem = ((size_t)rank * AF_CD_TOK + AF_CD_SLICES * AF_CD_TOK * 32) * sizeof(float);
    af_launch(channel_decay_few_kernel, dim3((n + 31) / 32), dim3(32 * AF_CD_SLICES), smem, stream, alpha, proj, ld, off_low,
              w2t, bias, rank, n, n_tokens, 1.f / tau);
    AF_CHECK_LAUNCH("af_channel_decay");
  }
  const dim3 grid((n + 127) / 128, (n_tokens + AF_CD_TOK - 1) / AF_CD_TOK);
  AF_REQUIRE(grid.y < 65536, "af_channel_decay: too many tokens for one grid");
  af_launch(channel_decay_kernel, grid, dim3(128), (size_t)rank * AF_CD_TOK * sizeof(float), stream, alpha, proj, ld,
            off_low, w2t, bias, rank, n, n_tokens, 1.f / tau);
  AF_CHECK_LAUNCH("af_channel_decay");
}

// ---------------------------------------------------------------- a long prompt's scan, chunks side by side

// The recurrence S <- diag(w_t) S + k_t v_t^T is linear in S, so a sequence can be cut into chunks that are scanned
// side by side, each from a zero state (state_scan over the chunks as if they were sequences: that gives
// o_local_t = S_local_t^T q_t and every chunk's final local state B), and joined afterwards, all in 32 bits:
//   cumulate   A_t = prod of w_s over the chunk's tokens s <= t                       (per key channel)
//   carry      S_in(first chunk) = the sequence's cached state; S_in(c + 1) = diag(A_end(c)) S_in(c) + B(c);
//              the last one is the sequence's new cached state
//   correct    o_t = o_local_t + S_in(chunk of t)^T (q_t * A_t)
// No quotient of decays is taken anywhere, so a channel that forgets quickly only drives its A towards zero.
// plan (int32, made on the host once a step): chunk_starts [n_chunks + 1] rows; seq_first_chunk [n_seqs + 1];
// tiles [n_tiles][3] = (first row, rows (<= 32), chunk).

__global__ void __launch_bounds__(128)
chunk_cumulate_kernel(float* __restrict__ A, const float* __restrict__ w, long long w_ts, const int* __restrict__ chunk_starts,
                      int n) {
  pdl_launch_dependents();
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int first = chunk_starts[blockIdx.y], last = chunk_starts[blockIdx.y + 1];
  pdl_wait();
  if (c >= n) return;
  float p = 1.f;
#pragma unroll 8
  for (int t = first; t < last; ++t) {
    p *= w[(size_t)t * w_ts + c];
    A[(size_t)t * n + c] = p;
  }
}

// One thread a state element (head, value column, key channel); blockIdx.y = sequence.  `local` holds B(c) on entry
// and S_in(c) on exit.
__global__ void __launch_bounds__(256)
chunk_carry_kernel(float* __restrict__ local, float* __restrict__ state, const float* __restrict__ A,
                   const int* __restrict__ chunk_starts, const int* __restrict__ seq_first_chunk,
                   const int* __restrict__ slots, int heads, int dk, int dv) {
  pdl_launch_dependents();
  const size_t per = (size_t)heads * dv * dk;
  const size_t e = (size_t)blockIdx.x * 256 + threadIdx.x;
  const int b = blockIdx.y;
  const int slot = slots[b];
  const int c0 = seq_first_chunk[b], c1 = seq_first_chunk[b + 1];
  pdl_wait();
  if (e >= per || slot < 0) return;
  const int ch = (int)(e % dk);
  const int h = (int)(e / ((size_t)dv * dk));
  const int n = heads * dk;
  float S = state[(size_t)slot * per + e];
  for (int c = c0; c < c1; ++c) {
    const float B = local[(size_t)c * per + e];
    const float a = A[(size_t)(chunk_starts[c + 1] - 1) * n + h * dk + ch];
    local[(size_t)c * per + e] = S;
    S = fmaf(a, S, B);
  }
  state[(size_t)slot * per + e] = S;
}

// Block (x, y, z) = (32 value columns, head, tile of up to 32 tokens of one chunk); 256 threads: thread (j, r) owns
// column j of tokens r, r + 8, r + 16, r + 24.  The key channels go through shared memory 64 at a time.
__global__ void __launch_bounds__(256)
chunk_correct_kernel(float* __restrict__ out, long long out_ts, const float* __restrict__ q, long long q_ts,
                     const float* __restrict__ A, const float* __restrict__ s_in, const int* __restrict__ tiles, int heads,
                     int dk, int dv) {
  pdl_launch_dependents();
  __shared__ float Ss[32][65];
  __shared__ float Qs[32][64];
  const int j = threadIdx.x & 31, r = threadIdx.x >> 5;
  const int j0 = blockIdx.x * 32, h = blockIdx.y;
  const int row0 = tiles[3 * blockIdx.z], rows = tiles[3 * blockIdx.z + 1], chunk = tiles[3 * blockIdx.z + 2];
  const int n = heads * dk;
  const float* S = s_in + (((size_t)chunk * heads + h) * dv) * dk;
  pdl_wait();
  q = pdl_fresh(q);
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int c0 = 0; c0 < dk; c0 += 64) {
    for (int i = threadIdx.x; i < 32 * 64; i += 256) {
      const int jj = i >> 6, cc = i & 63;
      Ss[jj][cc] = (j0 + jj < dv && c0 + cc < dk) ? S[(size_t)(j0 + jj) * dk + c0 + cc] : 0.f;
      const int tt = jj;                              // (the same index walks the tile's tokens)
      float v = 0.f;
      if (tt < rows && c0 + cc < dk) {
        const size_t t = (size_t)(row0 + tt);
        v = q[t * q_ts + h * dk + c0 + cc] * A[t * n + h * dk + c0 + cc];
      }
      Qs[tt][cc] = v;
    }
    __syncthreads();
#pragma unroll 16
    for (int cc = 0; cc < 64; ++cc) {
      const float s = Ss[j][cc];
#pragma unroll
      for (int u = 0; u < 4; ++u) acc[u] = fmaf(s, Qs[r + 8 * u][cc], acc[u]);
    }
    __syncthreads();
  }
  if (j0 + j >= dv) return;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int tt = r + 8 * u;
    if (tt < rows) out[(size_t)(row0 + tt) * out_ts + h * dv + j0 + j] += acc[u];
  }
}

// After af_state_scan over the chunks (rule CHANNEL, `local` [n_chunks, heads, dv, dk] as its zeroed state): join them.
// A: scratch [n_tokens, heads * dk].
AF_EXPORT int af_chunk_join(float* out, long long out_ts, const float* q, long long q_ts, const float* w, long long w_ts,
                            float* A, float* local, float* state, const int* chunk_starts, const int* seq_first_chunk,
                            const int* tiles, const int* slots, int n_chunks, int n_seqs, int n_tiles, int heads, int dk,
                            int dv, cudaStream_t stream) {
  if (n_chunks == 0) return 0;
  AF_REQUIRE(n_chunks > 0 && n_seqs > 0 && n_tiles > 0 && heads > 0 && dk > 0 && dv > 0, "af_chunk_join: bad sizes");
  AF_REQUIRE(n_chunks < 65536 && n_seqs < 65536 && n_tiles < 65536 && heads < 65536,
             "af_chunk_join: too many chunks, sequences, tiles or heads for one grid");
  const int n = heads * dk;
  af_launch(chunk_cumulate_kernel, dim3((n + 127) / 128, n_chunks), dim3(128), 0, stream, A, w, w_ts, chunk_starts, n);
  AF_COUNT_LAUNCH("af_chunk_join");
  const size_t per = (size_t)heads * dv * dk;
  af_launch(chunk_carry_kernel, dim3((unsigned)((per + 255) / 256), n_seqs), dim3(256), 0, stream, local, state,
            (const float*)A, chunk_starts, seq_first_chunk, slots, heads, dk, dv);
  AF_COUNT_LAUNCH("af_chunk_join");
  af_launch(chunk_correct_kernel, dim3((dv + 31) / 32, heads, n_tiles), dim3(256), 0, stream, out, out_ts, q, q_ts,
            (const float*)A, (const float*)local, tiles, heads, dk, dv);
  AF_CHECK_LAUNCH("af_chunk_join");
}
