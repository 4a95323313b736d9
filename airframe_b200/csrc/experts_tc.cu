// The products of routed experts on the 5th-generation tensor cores (bfloat16): a grouped matrix product over
// rows that are sorted by expert.
//
//   DUAL   mid[row, f] = act(s (x[row] . gate_e[f]), s (x[row] . up_e[f])) * post     (bfloat16, sorted rows)
//   else   out[choice, token, f] = mid[row] . down_e[f]                               (float, scattered by pair)
//
// A tile is 128 output features of one expert (the tcgen05 "A" operand: the TMEM lanes) by up to BN sorted rows of
// that expert (TMEM columns).  The plan (expert_plan) lists the row tiles: (expert, first sorted row, rows); a TMA
// box of BN rows starts at the tile's first row wherever that lies (only the innermost coordinate of a copy must
// be aligned), the instruction's N is the tile's rows rounded up to 16, and rows of the box beyond the tile's own
// (the next expert's, or zeros beyond the end) are computed at most up to that rounding and never stored.  The
// experts' matrices are one [experts * N, K] tensor: the tile's weight rows begin at expert * N + 128 * wt, and
// rows it reads beyond its expert's last are masked in the epilogue.  DUAL keeps two accumulators (gate and up
// of the same features), so the activation needs no exchange between lanes.
//
//   warp 0      TMA producer (one lane)
//   warp 1      TMEM allocation, MMA issue (one lane), TMEM release
//   warps 2..5  epilogue: TMEM -> registers -> global
//
// GATES is the same grouped product put to another use: the two gates of a gated linear recurrence, whose
// matrices are block-diagonal.  An "expert" is a block of channels, every block takes all rows, its columns of
// the input rows begin at block * K, and the epilogue turns the two sums into what the scan wants:
//   r = sigmoid(. + ba), i = sigmoid(. + bi), a = exp(-rate r):  decay = 1 - a,  input = sqrt(1 - a^2) i u.
//
// A block walks the tiles blockIdx.x, + gridDim.x, ... (feature tile fastest: blocks that run together share a
// row tile in L2); the number of row tiles is read from the plan on the device, so the host never waits for it.
// Every wait on an mbarrier is bounded in time; one that runs out sets the error word, lets copies land, frees
// the TMEM and returns.
#include "umma.cuh"

namespace {

constexpr int EX_BM = 128;
constexpr int EX_BK = 64;
constexpr int EX_THREADS = 192;

__host__ __device__ constexpr int ex_stage_bytes(int bn, int nacc) { return nacc * EX_BM * EX_BK * 2 + bn * EX_BK * 2; }
__host__ __device__ constexpr int ex_stages(int bn, int nacc) {
  // few rows: the weights stream through once, two blocks share an SM; many rows: a block per SM
  int s = (bn <= 64 ? 100 * 1024 : 192 * 1024) / ex_stage_bytes(bn, nacc);
  return s > 8 ? 8 : s;
}
__host__ __device__ constexpr int ex_tmem_cols(int bn, int nacc) { return nacc * bn < 32 ? 32 : nacc * bn; }

struct ExArgs {
  void* out;
  int N, K;                 // output features of an expert; the products' length
  int n_rows, n_tokens, top;
  int tiles_w;              // feature tiles of an expert
  int max_row_tiles;        // room of the plan (without a plan: the row tiles themselves)
  const int* perm;          // sorted row -> pair (null: the rows are the pairs)
  const int* plan;          // [0] row tiles in use, then (expert, first sorted row, rows) each (null: one expert)
  const float* pair_weight; // DUAL: s per pair (null: 1)
  const float* scale_out;   // DUAL: post per token (null: 1)
  float limit;
  int* err;
  // GATES only
  int uniform;              // every expert takes all rows (no plan): row tiles of BN rows, expert by expert
  float* out2;              // input [rows, experts * N]; out is decay
  const float* u;           // [rows, experts * N] 32-bit, what the bfloat16 rows were rounded from
  long long ld_u;           // experts * N
  const float* ba;
  const float* bi;
  const float* rate;
};

enum { EX_DOWN = 0, EX_ACT = 1, EX_GATES = 2, EX_GELU = 3 };
__host__ __device__ constexpr int ex_accs(int epi) { return epi == EX_ACT || epi == EX_GATES ? 2 : 1; }

__device__ __forceinline__ float ex_act(float g, float u, float limit) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  // g sigmoid(1.702 g) with sigmoid(z) = (1 + tanh(z / 2)) / 2: one special-function operation; the result is
  // rounded to bfloat16
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.851f * g));
  return 0.5f * g * (1.f + t) * (u + 1.f);
}

__device__ __forceinline__ void ex_tile(const ExArgs& a, int row_tile, int bn, int* expert, int* row0, int* rows) {
  if (a.plan != nullptr) {
    *expert = __ldcg(a.plan + 1 + 3 * row_tile);
    *row0 = __ldcg(a.plan + 2 + 3 * row_tile);
    *rows = __ldcg(a.plan + 3 + 3 * row_tile);
  } else if (a.uniform) {
    const int per = (a.n_rows + bn - 1) / bn;
    *expert = row_tile / per;
    *row0 = (row_tile % per) * bn;
    *rows = min(bn, a.n_rows - *row0);
  } else {
    *expert = 0;
    *row0 = row_tile * bn;
    *rows = min(bn, a.n_rows - *row0);
  }
}

template <int BN, int EPI>
__global__ void __launch_bounds__(EX_THREADS, BN <= 64 ? 2 : 1)
expert_rows_tc_kernel(const __grid_constant__ CUtensorMap map_w0, const __grid_constant__ CUtensorMap map_w1,
                      const __grid_constant__ CUtensorMap map_x, ExArgs a) {
  constexpr bool DUAL = ex_accs(EPI) == 2;
  constexpr bool GATES = EPI == EX_GATES;
  constexpr bool SINGLE = EPI == EX_GELU;        // one matrix with the exact GELU behind it, rows out like DUAL's
  constexpr int NACC = ex_accs(EPI);
  constexpr int XB = BN < 64 ? BN : 64;          // rows of a box of the input rows: a tile fetches as many boxes as hold its rows
  constexpr int STAGES = ex_stages(BN, NACC);
  constexpr int A_BYTES = EX_BM * EX_BK * 2;
  constexpr int STAGE_BYTES = ex_stage_bytes(BN, NACC);
  constexpr int COLS = ex_tmem_cols(BN, NACC);
  static_assert(STAGES >= 2, "at least two stages");

  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full[STAGES], empty[STAGES], acc_full, acc_empty;
  __shared__ uint32_t tmem_base_s;
  __shared__ int give_up_s;
  volatile int* give_up = &give_up_s;

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_kb = (a.K + EX_BK - 1) / EX_BK;
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w0) : "memory");
    if (DUAL) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w1) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(&acc_full, 1);
    mbar_init(&acc_empty, 4);   // one arrival an epilogue warp
    give_up_s = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                 "r"((uint32_t)COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;

  // the plan, the permutation and the rows come from the kernels in front
  pdl_wait();
  int row_tiles = a.max_row_tiles;
  if (a.plan != nullptr) row_tiles = min(__ldcg(a.plan), a.max_row_tiles);
  const int n_tiles = row_tiles * a.tiles_w;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      for (int tile = blockIdx.x; tile < n_tiles && !*give_up; tile += gridDim.x) {
        int expert, row0, rows;
        ex_tile(a, tile / a.tiles_w, BN, &expert, &row0, &rows);
        const int w_row = expert * a.N + (tile % a.tiles_w) * EX_BM;
        const int x_col = GATES ? expert * a.K : 0;
        const int boxes = (min(rows, BN) + XB - 1) / XB;
        bool ok = true;
        for (int kb = 0; kb < total_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (it >= STAGES && !mbar_wait(&empty[s], ph ^ 1, give_up)) {
            ok = false;
            break;
          }
          unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
          mbar_expect_tx(&full[s], NACC * A_BYTES + boxes * XB * EX_BK * 2);
          const int k = kb * EX_BK;
          tma_load_2d(st, &map_w0, k, w_row, &full[s]);
          if (DUAL) tma_load_2d(st + A_BYTES, &map_w1, k, w_row, &full[s]);
          for (int b = 0; b < boxes; ++b)
            tma_load_2d(st + NACC * A_BYTES + b * XB * EX_BK * 2, &map_x, x_col + k, row0 + b * XB, &full[s]);
        }
        if (!ok) break;
      }
      if (*give_up) grace_period();
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      int it = 0, round = 0;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++round) {
        int expert, row0, rows;
        ex_tile(a, tile / a.tiles_w, BN, &expert, &row0, &rows);
        const int n_eff = min(BN, max(16, (rows + 15) & ~15));
        const uint32_t idesc = umma_idesc(n_eff);
        if (round > 0 && !mbar_wait(&acc_empty, (round - 1) & 1, give_up)) {
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (int kb = 0; kb < total_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full[s], ph, give_up)) {
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t st = smem_u32(tiles + (size_t)s * STAGE_BYTES);
          const uint64_t db = umma_desc(st + NACC * A_BYTES);
#pragma unroll
          for (int k = 0; k < EX_BK / 16; ++k) {
            const uint32_t accum = (kb > 0 || k > 0) ? 1u : 0u;
#pragma unroll
            for (int acc = 0; acc < NACC; ++acc)
              umma_f16(tmem_base + acc * BN, umma_desc(st + acc * A_BYTES) + 2 * k, db + 2 * k, idesc, accum);
          }
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(&acc_full);
      }
    }
  } else {
    const int quarter = warp & 3;          // this warp reads TMEM lanes [32 * quarter, + 32)
    constexpr int CW = BN >= 32 ? 32 : 16;
    int round = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++round) {
      int expert, row0, rows;
      ex_tile(a, tile / a.tiles_w, BN, &expert, &row0, &rows);
      const int f = (tile % a.tiles_w) * EX_BM + quarter * 32 + lane;
      if (!mbar_wait(&acc_full, round & 1, give_up)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
      const int n_chunks = (min(rows, BN) + CW - 1) / CW;
#pragma unroll 1
      for (int ch = 0; ch < n_chunks; ++ch) {
        const int c0 = ch * CW;
        float g[CW], u[DUAL ? CW : 1];
        if constexpr (CW == 32) {
          tmem_ld32(lane_base + c0, g);
          if constexpr (DUAL) tmem_ld32(lane_base + BN + c0, u);
        } else {
          tmem_ld16(lane_base + c0, g);
          if constexpr (DUAL) tmem_ld16(lane_base + BN + c0, u);
        }
        if constexpr (GATES) {
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (ch == n_chunks - 1) {
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty);
          }
          if (f < a.N) {
            const int col = expert * a.N + f;
            const size_t ldu = (size_t)a.ld_u;
            const float ab = __ldg(a.ba + col), ib = __ldg(a.bi + col), rt = __ldg(a.rate + col);
            const int n = min(CW, rows - c0);
            float uv[CW];
#pragma unroll
            for (int j = 0; j < CW; ++j) uv[j] = j < n ? __ldcg(a.u + (size_t)(row0 + c0 + j) * ldu + col) : 0.f;
#pragma unroll
            for (int j = 0; j < CW; ++j) {
              if (j >= n) continue;
              const float r = __fdividef(1.f, 1.f + expf(-(g[j] + ab)));
              const float i = __fdividef(1.f, 1.f + expf(-(u[j] + ib)));
              const float d = -expm1f(-rt * r);                       // 1 - a, a = exp(-rate r)
              const size_t at = (size_t)(row0 + c0 + j) * ldu + col;
              static_cast<float*>(a.out)[at] = d;
              a.out2[at] = sqrtf(d * (2.f - d)) * i * uv[j];          // 1 - a^2 = (1 - a)(1 + a)
            }
          }
          continue;
        }
        // what the chunk's rows need besides the sums: lane l fetches it for row c0 + l
        const int r = c0 + lane;
        int pair = -1;
        if (lane < CW && r < rows) pair = a.perm != nullptr ? __ldcg(a.perm + row0 + r) : row0 + r;
        float s_l = 1.f, post_l = 1.f;
        int dst_l = -1;                                   // (DOWN: the row of out, top * n_tokens of them)
        if (pair >= 0) {
          if constexpr (DUAL || SINGLE) {
            if (a.pair_weight != nullptr) s_l = __ldcg(a.pair_weight + pair);
            if (a.scale_out != nullptr) post_l = __ldcg(a.scale_out + pair / a.top);
          } else {
            dst_l = (pair % a.top) * a.n_tokens + pair / a.top;
          }
        }
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (ch == n_chunks - 1) {
          // everything of this tile is in registers: the next tile's products may start
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty);
        }
        const int n = min(CW, rows - c0);                 // (sorted rows: the chunk's first n are the tile's)
        if constexpr (DUAL || SINGLE) {
          const bool scaled = a.pair_weight != nullptr, posted = a.scale_out != nullptr;
          __nv_bfloat16* o = static_cast<__nv_bfloat16*>(a.out) + (size_t)(row0 + c0) * a.N + f;
#pragma unroll
          for (int j = 0; j < CW; ++j) {
            const float s = scaled ? __shfl_sync(0xffffffffu, s_l, j) : 1.f;
            const float post = posted ? __shfl_sync(0xffffffffu, post_l, j) : 1.f;
            if (j >= n || f >= a.N) continue;
            if constexpr (SINGLE)       // (the weight stands behind the activation: it is the expert's output that is weighed)
              o[(size_t)j * a.N] = __float2bfloat16_rn(0.5f * g[j] * (1.f + erff(g[j] * 0.70710678118654752f)) * s * post);
            else
              o[(size_t)j * a.N] = __float2bfloat16_rn(ex_act(s * g[j], s * u[j], a.limit) * post);
          }
        } else {
#pragma unroll
          for (int j = 0; j < CW; ++j) {
            const int dst = __shfl_sync(0xffffffffu, dst_l, j);
            if (dst < 0 || f >= a.N) continue;
            static_cast<float*>(a.out)[(size_t)dst * a.N + f] = g[j];
          }
        }
      }
      if (n_chunks == 0) {      // (a tile without rows: never planned, but the accumulators must be handed back)
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty);
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)COLS));
  }
  if (threadIdx.x == 0 && give_up_s && a.err) atomicExch(a.err, 1);
}

template <int BN, int EPI>
int ex_launch(const CUtensorMap& m0, const CUtensorMap& m1, const CUtensorMap& mx, const ExArgs& a, cudaStream_t stream) {
  constexpr int NACC = ex_accs(EPI);
  constexpr int smem = ex_stages(BN, NACC) * ex_stage_bytes(BN, NACC) + 1024;
  static bool configured[AF_MAX_DEVICES] = {};
  const int dev = af_current_device();
  if (dev < 0) return -1;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(expert_rows_tc_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return af_fail((int)e, "expert_rows_tc: %s", cudaGetErrorString(e));
    configured[dev] = true;
  }
  const int sms = af_sm_count();
  if (sms <= 0) return -1;
  const long long tiles = (long long)a.max_row_tiles * a.tiles_w;
  const long long most = BN <= 64 ? tiles : (tiles < sms ? tiles : sms);   // few rows: a block per tile
  af_launch(expert_rows_tc_kernel<BN, EPI>, dim3((unsigned)most), dim3(EX_THREADS), smem, stream, m0, m1, mx, a);
  AF_CHECK_LAUNCH("af_expert_rows_tc");
}

template <int EPI>
int ex_launch_bn(int bn, const CUtensorMap& m0, const CUtensorMap& m1, const CUtensorMap& mx, const ExArgs& a,
                 cudaStream_t s) {
  switch (bn) {
    case 16: return ex_launch<16, EPI>(m0, m1, mx, a, s);
    case 32: return ex_launch<32, EPI>(m0, m1, mx, a, s);
    case 64: return ex_launch<64, EPI>(m0, m1, mx, a, s);
    case 128: return ex_launch<128, EPI>(m0, m1, mx, a, s);
    case 256: return ex_launch<256, EPI>(m0, m1, mx, a, s);
  }
  return af_fail(-1, "af_expert_rows_tc: row tile %d", bn);
}

}  // namespace

// The sorted rows' products on the tensor cores.  a [n_rows, K] bfloat16 in sorted order (w1 given: the rows that
// the pairs' tokens name, gathered; else the first product's output); w0, w1 [experts, N, K] bfloat16; tile: the
// plan's row tile (16, 32, 64, 128 or 256; at most so many rows a plan entry).  K a multiple of 8, bases 16-byte
// aligned.  act 1 (no w1): out[sorted row] = gelu(a w0[e]^T) * s * post with the exact (erf) GELU, rows of the
// compute dtype like the two-matrix form's.  Otherwise as af_expert_rows.
AF_EXPORT int af_expert_rows_tc(void* out, const void* a, const void* w0, const void* w1, int n_experts, const int* perm,
                                const int* plan, const float* pair_weight, const float* scale_out, int n_rows,
                                int n_tokens, int top, int max_tiles, int tile, int N, int K, float limit, int act,
                                int* err, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  AF_REQUIRE(n_rows > 0 && n_tokens > 0 && top >= 1 && N > 0 && K > 0 && n_experts > 0, "af_expert_rows_tc: bad sizes");
  AF_REQUIRE((plan == nullptr) == (perm == nullptr), "af_expert_rows_tc: a plan and its permutation, or neither");
  AF_REQUIRE(plan != nullptr || n_experts == 1, "af_expert_rows_tc: several experts need a plan");
  AF_REQUIRE(n_rows == n_tokens * top, "af_expert_rows_tc: %d rows for %d tokens with %d choices", n_rows, n_tokens, top);
  AF_REQUIRE(K % 8 == 0, "af_expert_rows_tc: K %d must be a multiple of 8", K);
  AF_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)w0 & 15) == 0 && ((uintptr_t)w1 & 15) == 0,
             "af_expert_rows_tc: operands must be 16-byte aligned");
  AF_REQUIRE((long long)n_experts * N < 0x7fffffffll, "af_expert_rows_tc: too many weight rows");
  CUtensorMap m0, m1, mx;
  int rc = af_make_map_bf16(&m0, w0, (long long)n_experts * N, K, K, EX_BM);
  if (rc) return rc;
  rc = af_make_map_bf16(&m1, w1 != nullptr ? w1 : w0, (long long)n_experts * N, K, K, EX_BM);
  if (rc) return rc;
  rc = af_make_map_bf16(&mx, a, n_rows, K, K, tile < 64 ? tile : 64);
  if (rc) return rc;
  ExArgs args{out, N, K, n_rows, n_tokens, top, (N + EX_BM - 1) / EX_BM,
              plan != nullptr ? max_tiles : (n_rows + tile - 1) / tile, perm, plan, pair_weight, scale_out, limit, err};
  AF_REQUIRE(args.max_row_tiles > 0, "af_expert_rows_tc: no tiles");
  AF_REQUIRE(act == 0 || (act == 1 && w1 == nullptr), "af_expert_rows_tc: the exact GELU stands behind one matrix");
  if (w1 != nullptr) return ex_launch_bn<EX_ACT>(tile, m0, m1, mx, args, stream);
  if (act == 1) return ex_launch_bn<EX_GELU>(tile, m0, m1, mx, args, stream);
  return ex_launch_bn<EX_DOWN>(tile, m0, m1, mx, args, stream);
}

// The gates of a gated linear recurrence on the tensor cores: with the channels in `blocks` equal parts of bw,
// u16 [n_rows, blocks * bw] bfloat16 (the rounding of u), wa, wi [blocks, bw, bw] bfloat16 ([out, in]):
//   r = sigmoid(wa_b u_b + ba), i = sigmoid(wi_b u_b + bi), a = exp(-rate r), decay = 1 - a, input = sqrt(1 - a^2) i u
// with the sums in 32 bits and everything behind them in 32 bits from the 32-bit u.  bw a multiple of 8.
AF_EXPORT int af_gate_rows_tc(float* decay, float* input, const float* u, const void* u16, const void* wa, const void* wi,
                              const float* ba, const float* bi, const float* rate, int n_rows, int blocks, int bw,
                              int* err, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  AF_REQUIRE(n_rows > 0 && blocks > 0 && bw > 0 && bw % 8 == 0, "af_gate_rows_tc: %d blocks of %d channels", blocks, bw);
  AF_REQUIRE(((uintptr_t)u16 & 15) == 0 && ((uintptr_t)wa & 15) == 0 && ((uintptr_t)wi & 15) == 0,
             "af_gate_rows_tc: operands must be 16-byte aligned");
  // (the products are short and the epilogue is long: small row tiles, a block each, two blocks an SM)
  const int tile = n_rows <= 16 ? 16 : n_rows <= 32 ? 32 : 64;
  const long long width = (long long)blocks * bw;
  CUtensorMap m0, m1, mx;
  int rc = af_make_map_bf16(&m0, wa, width, bw, bw, EX_BM);
  if (rc) return rc;
  rc = af_make_map_bf16(&m1, wi, width, bw, bw, EX_BM);
  if (rc) return rc;
  rc = af_make_map_bf16(&mx, u16, n_rows, width, width, tile < 64 ? tile : 64);
  if (rc) return rc;
  ExArgs args{decay, bw, bw, n_rows, n_rows, 1, (bw + EX_BM - 1) / EX_BM, blocks * ((n_rows + tile - 1) / tile),
              nullptr, nullptr, nullptr, nullptr, 0.f, err};
  args.uniform = 1;
  args.out2 = input;
  args.u = u;
  args.ld_u = width;
  args.ba = ba;
  args.bi = bi;
  args.rate = rate;
  return ex_launch_bn<EX_GATES>(tile, m0, m1, mx, args, stream);
}
