// bf16 matrix product on the 5th-generation tensor cores: C[M, N] = X[M, K] . W[N, K]^T (+ bias), float32 accumulation.
//
// One kernel serves prompt portions and decoded tokens. Both operands are K-major in global memory, so either can be
// the 128-row operand of `tcgen05.mma`:
//   rows mode  (many tokens): the 128 TMEM lanes are token rows, the instruction's N (BN = 64..256) are output features;
//   swap mode  (few tokens):  the 128 TMEM lanes are output features (rows of W, the operand that has to be streamed
//                             from HBM once), the instruction's N (BN = 16..128) are the token rows; the tile is stored
//                             transposed. Nothing is padded to 128 tokens. (The reference's decode GEMM swaps operands the
//                             same way on sm_90a wgmma: fusezap/device/cuda_kernels/wgmma.py:182-317.)
// Rows mode is persistent: the output tiles are walked token tiles fastest (so the CTAs running at one time share a few
// weight tiles in L2), the MMA lane alternates between two TMEM accumulators, and the epilogue warps store one tile
// while the next one is being computed. Where the token rows fill them, a PAIR of CTAs (a cluster of two) works on each
// 256 x 256 tile with `tcgen05.mma.cta_group::2` (`gemm_tc_rows_pair_kernel`); else one CTA per SM walks 128 x 256 tiles
// (`gemm_tc_rows_kernel`). Products of a few hundred rows with too few tiles for the SMs have their tiles' K ranges cut
// over a cluster (`gemm_tc_rows_split_kernel`, in both forms). Swap mode: a CTA computes one 128 x BN tile over one
// range of K:
//   warp 0  one lane issues the TMA loads (cp.async.bulk.tensor.2d, 128-byte swizzle, 64 k per stage) into a ring of
//           shared-memory stages guarded by full/empty mbarriers; no multicast;
//   warp 1  allocates the TMEM accumulator; one lane issues tcgen05.mma (128 x BN x 16, 4 per stage) and commits each
//           stage's completion to its empty barrier, the last one to the accumulator-ready barrier;
//   warps 2-5  read the accumulator with tcgen05.ld (each warp its own 32 lanes), add the bias and store.
// Split K (swap mode; the count is chosen from N and K only, never from M): the splits of a tile form one thread-block
// cluster. Each CTA leaves its float32 partial tile in its own shared memory; after a cluster barrier CTA r adds, for
// the columns r, r + S, ..., the partials of all splits in split order 0, 1, 2, ... through distributed shared memory and
// stores the result. The sum has one fixed order (as the reference's split-K has: wgmma.py:209-239) and no partial ever
// goes to global memory. Waits on this CTA's own mbarriers are bounded by a time limit after which the kernel sets an
// error bit and leaves; the cluster barriers are hardware barriers, not spins.
// Epilogues besides bias + store: SwiGLU over weight rows packed as [64 gate | 64 up] blocks (both modes); for few
// tokens the rotation of the q and k heads with the write of k and v into the paged cache, and a per-tile argmax that
// stores no products at all (the lm_head of a greedy step).
#include "umma.cuh"

namespace {
using namespace fztma;
using namespace fzumma;

constexpr int BM = 128;           // TMEM lanes = rows of the 128-row operand
constexpr int BK = 64;            // k per stage: 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;  // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue
constexpr int PAIR_THREADS_G = 320;      // the many-token kernels: warps 2..9 epilogue (two per quarter of the tensor-memory lanes)

// ---------------------------------------------------------------------------------------------- cluster helpers
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The float at shared-memory address `addr` of the cluster's CTA `rank`
__device__ __forceinline__ float ld_dsmem(uint32_t addr, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
  // (volatile keeps it behind the cluster barrier, itself a volatile asm; no memory clobber, so that the loads of the
  // next column may be issued before this column's result is stored)
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote));
  return v;
}
__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.0f + __expf(-g)) * u; }
// (value, index) order of numpy.argmax: a NaN is the maximum, among equals the lower index wins; index 0x7fffffff: none
__device__ __forceinline__ bool am_better(float v, int i, float bv, int bi) {
  if (i == 0x7fffffff) return false;
  if (bi == 0x7fffffff) return true;
  const bool vn = isnan(v), bn = isnan(bv);
  if (vn != bn) return vn;
  if (vn) return i < bi;
  if (v != bv) return v > bv;
  return i < bi;
}

struct Params {
  float* c_f32;            // exactly one of c_f32 / c_bf16 is set
  __nv_bfloat16* c_bf16;
  const float* bias;       // over output features, may be null
  int* err;
  int rows;                // token rows (M of the product)
  int feats;               // output features (N of the product)
  int K;
  int swap;                // 1: lanes are features, columns are token rows
  int splits;
  int stages;
  int vec_ok;              // rows mode: C rows are 16-byte aligned, so full groups of 16 columns go out as vectors
  int swiglu;              // W holds [64 gate rows | 64 up rows] blocks: store silu(gate) * up as bf16 [rows, feats / 2]
  // rope != 0 (swap mode, hd divides 128): the features are [q heads | k heads | v heads] of size hd; q and k are rotated
  // by the token's position, q goes to c_bf16 [rows, Hq * hd], k and v to the token's slot of the paged pool
  int rope;
  const float* cos_t;      // [max_len, hd / 2]
  const float* sin_t;
  const int* pos;          // [rows]
  const int* seq_row;      // [rows], negative: padding (q zeros, nothing stored)
  const int* table;        // [requests, mb] block table of the layer's cache group
  int mb;
  __nv_bfloat16* k_pool;
  __nv_bfloat16* v_pool;
  long long page_stride;
  int page_size, write, Hq, Hkv, hd, max_len;
  // argmax != 0 (few tokens, no split): nothing is stored but, per token row and 128-feature tile, the largest value
  // and its feature index (numpy's order: a NaN is the maximum, the lower index wins among equals)
  int argmax;
  float* am_val;           // [rows][tiles]
  int* am_idx;
};

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  // stages of [A: 128 x 64 bf16][B: BN x 64 bf16], 1024-byte aligned for the swizzle
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
  uint64_t* full = (uint64_t*)(smem + (size_t)p.stages * STAGE_BYTES);
  uint64_t* empty = full + p.stages;
  uint64_t* acc_ready = empty + p.stages;
  uint32_t* tmem_slot = (uint32_t*)(acc_ready + 1);
  int* flag = (int*)(tmem_slot + 1);     // [0]: this CTA arrived last at its tile  [1]: a wait gave up

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_a = blockIdx.x, tile_b = blockIdx.y, split = blockIdx.z;
  const int kblocks = (p.K + BK - 1) / BK;
  const int kb0 = (int)((long long)kblocks * split / p.splits), kb1 = (int)((long long)kblocks * (split + 1) / p.splits);
  const int nkb = kb1 - kb0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(acc_ready, 1);
    flag[0] = 0; flag[1] = 0;
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = *tmem_slot;
  fz_grid_launch_dependents();
  // The rotation epilogue needs, of every token column this thread will finish, the request's row, the position, the
  // page and the angles: loads that depend on one another and on nothing a kernel before this one writes (the host
  // packed the step's metadata before the step began). They are asked for now, by the epilogue warps that would
  // otherwise only wait, instead of column by column at the end. Measured with two engines alternating in one process:
  // a batch-1 decode step of 32 layers 3.304 -> 3.210 ms; batch 8 and 32 unchanged (looking up eight columns ahead
  // instead of two was no better there either, and slower at batch 4 and 32).
  constexpr int PRE = 2;      // columns per thread that are looked up ahead; further ones are looked up in the loop
  int pre_row[PRE], pre_ps[PRE], pre_page[PRE];
  float pre_cos[PRE], pre_sin[PRE];
  if (p.rope && warp >= 2) {
    const int rank0 = p.splits > 1 ? (int)cluster_rank() : 0, cols0 = min(BN, p.rows - tile_b * BN);
    const int feat = tile_a * BM + (warp & 3) * 32 + lane, head = feat / p.hd, j = feat - head * p.hd, half = p.hd >> 1;
#pragma unroll
    for (int i = 0; i < PRE; ++i) {
      const int c = rank0 + i * p.splits;
      pre_row[i] = c < cols0 ? p.seq_row[tile_b * BN + c] : -1;
      pre_ps[i] = c < cols0 ? p.pos[tile_b * BN + c] : 0;
    }
#pragma unroll
    for (int i = 0; i < PRE; ++i) {
      const bool live = pre_row[i] >= 0 && pre_ps[i] >= 0 && pre_ps[i] < p.max_len && feat < p.feats;
      pre_page[i] = (live && p.write && head >= p.Hq) ? p.table[(size_t)pre_row[i] * p.mb + pre_ps[i] / p.page_size] : -1;
      const bool turn = live && head < p.Hq + p.Hkv && j < half;
      pre_cos[i] = turn ? p.cos_t[(size_t)pre_ps[i] * half + j] : 0.f;
      pre_sin[i] = turn ? p.sin_t[(size_t)pre_ps[i] * half + j] : 0.f;
    }
  }
  if (warp != 0) fz_grid_wait();    // warp 0 waits after it has requested the first weight stages

  if (warp == 0) {
    if (lane == 0) {
      // The weight operand does not depend on the kernel before this one: its first stages are requested before the
      // wait on that kernel, so the weights stream in while it finishes. (swap mode: A holds the weights; rows mode: B.)
      const uint64_t stream_once = l2_evict_first();
      auto load_weights = [&](int i, int s) {
        uint8_t* sa = smem + (size_t)s * STAGE_BYTES;
        // swap mode streams every weight once per step: it should leave L2 before the activations, which are read again
        if (p.swap) tma_load_2d_u32_hint(smem_u32(sa), &map_a, smem_u32(&full[s]), (kb0 + i) * BK, tile_a * BM, stream_once);
        else tma_load_2d(sa + A_BYTES, &map_b, &full[s], (kb0 + i) * BK, tile_b * BN);
      };
      auto load_activations = [&](int i, int s) {
        uint8_t* sa = smem + (size_t)s * STAGE_BYTES;
        if (p.swap) tma_load_2d(sa + A_BYTES, &map_b, &full[s], (kb0 + i) * BK, tile_b * BN);
        else tma_load_2d(sa, &map_a, &full[s], (kb0 + i) * BK, tile_a * BM);
      };
      const int early = nkb < p.stages ? nkb : p.stages;
      for (int i = 0; i < early; ++i) {
        mbar_expect_tx(&full[i], STAGE_BYTES);
        load_weights(i, i);
      }
      fz_grid_wait();
      for (int i = 0, s = 0, round = 0; i < nkb; ++i) {
        if (round > 0) {
          if (!mbar_wait(&empty[s], (round - 1) & 1)) { flag[1] = 1; break; }
          mbar_expect_tx(&full[s], STAGE_BYTES);
          load_weights(i, s);
        }
        load_activations(i, s);
        if (++s == p.stages) { s = 0; ++round; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN);
      bool ok = true;
      for (int i = 0, s = 0, round = 0; i < nkb && ok; ++i) {
        if (!mbar_wait(&full[s], round & 1)) { flag[1] = 1; ok = false; break; }
        tc_fence_after();
        const uint8_t* sa = smem + (size_t)s * STAGE_BYTES;
        const uint64_t da = desc_k_major(smem_u32(sa)), db = desc_k_major(smem_u32(sa + A_BYTES));
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)   // 32 bytes further along the swizzled row per 16 k
          umma_bf16(tmem_d, da + (uint64_t)(k * UMMA_K * 2 / 16), db + (uint64_t)(k * UMMA_K * 2 / 16), idesc,
                    (i > 0 || k > 0) ? 1u : 0u);
        umma_commit(&empty[s]);
        if (++s == p.stages) { s = 0; ++round; }
      }
      umma_commit(acc_ready);   // arrives when every MMA issued so far has finished (at once if none was issued)
    }
  } else {
    // ---- epilogue: 4 warps, warp w reads TMEM lanes 32 * (w % 4) ..
    const int quad = warp & 3;
    const int r = quad * 32 + lane;          // TMEM lane = row of the 128-row operand
    const bool ok = __all_sync(0xffffffffu, mbar_wait(acc_ready, 0));   // warp-uniform: tcgen05.ld is warp-wide
    if (!ok) flag[1] = 1;
    tc_fence_after();
    const int a_row = tile_a * BM + r;       // rows mode: token row; swap mode: output feature
    const int a_limit = p.swap ? p.feats : p.rows;
    const int b_limit = p.swap ? p.rows : p.feats;
    const int b0 = tile_b * BN;
    const uint32_t taddr = tmem_d + ((uint32_t)(quad * 32) << 16);
    const bool direct = p.splits == 1 && !p.swiglu && !p.rope;
    float* part = (float*)smem + r;          // split K: partial tile as [column][row] in the (now idle) stage buffers
    float v[16];
    auto store16 = [&](const float* x, int c) {   // columns c..c+15 of this thread's row, final values
      if (a_row >= a_limit) return;
      if (p.swap) {
        const float bv = p.bias ? p.bias[a_row] : 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int m = b0 + c + j;
          if (m < b_limit) {
            const float y = x[j] + bv;
            if (p.c_f32) p.c_f32[(size_t)m * p.feats + a_row] = y;
            else p.c_bf16[(size_t)m * p.feats + a_row] = __float2bfloat16_rn(y);
          }
        }
      } else if (p.vec_ok && b0 + c + 16 <= b_limit) {
        const int n = b0 + c;
        float y[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) y[j] = x[j] + (p.bias ? p.bias[n + j] : 0.f);
        if (p.c_f32) {
          float4* dst = (float4*)(p.c_f32 + (size_t)a_row * p.feats + n);
#pragma unroll
          for (int j = 0; j < 4; ++j) dst[j] = make_float4(y[4 * j], y[4 * j + 1], y[4 * j + 2], y[4 * j + 3]);
        } else {
          uint32_t w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(y[2 * j], y[2 * j + 1]);
            w[j] = *(const uint32_t*)&h;
          }
          uint4* dst = (uint4*)(p.c_bf16 + (size_t)a_row * p.feats + n);
          dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
          dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int n = b0 + c + j;
          if (n < b_limit) {
            const float y = x[j] + (p.bias ? p.bias[n] : 0.f);
            if (p.c_f32) p.c_f32[(size_t)a_row * p.feats + n] = y;
            else p.c_bf16[(size_t)a_row * p.feats + n] = __float2bfloat16_rn(y);
          }
        }
      }
    };
    if (ok) {
      for (int c = 0; c < BN; c += 16) {
        if (nkb > 0) tmem_ld16(taddr + (uint32_t)c, v);
        else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
        }
        if (p.argmax) {
          // the tile's logits go to the (idle) stage buffers as [token][feature], rows one float apart from a multiple of
          // the bank count, and are searched below
          const float bv = (p.bias && a_row < a_limit) ? p.bias[a_row] : 0.f;
          float* am = (float*)smem;                   // [BN][BM + 1]
#pragma unroll
          for (int j = 0; j < 16; ++j) am[(c + j) * (BM + 1) + r] = v[j] + bv;
        } else if (direct) store16(v, c);
        else {
#pragma unroll
          for (int j = 0; j < 16; ++j) part[(c + j) * BM] = v[j];
        }
      }
      if (p.argmax) {
        // 128 / BN threads share a token: each scans its part of the tile's 128 features in rising order (so the lower
        // index wins among equals), then the parts are merged in rising order
        asm volatile("bar.sync 1, 128;" ::: "memory");
        constexpr int TPC = BM / BN < 1 ? 1 : BM / BN;          // threads per token
        constexpr int SEG = BM / TPC;                            // features per thread
        const float* am = (const float*)smem;
        float* best_v = (float*)smem + BN * (BM + 1);            // [BN][TPC]
        int* best_i = (int*)(best_v + BN * TPC);
        const int col = r % BN, seg = r / BN;                    // (for BN = 128 every thread has a token of its own)
        float x = 0.f;
        int ix = 0x7fffffff;
        if (seg < TPC) {
          for (int i = 0; i < SEG; ++i) {
            const int f = seg * SEG + i, feat = tile_a * BM + f;
            if (feat < a_limit && am_better(am[col * (BM + 1) + f], feat, x, ix)) { x = am[col * (BM + 1) + f]; ix = feat; }
          }
          best_v[col * TPC + seg] = x;
          best_i[col * TPC + seg] = ix;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int m = b0 + col;
        if (seg == 0 && m < b_limit) {
          for (int sgm = 1; sgm < TPC; ++sgm)
            if (am_better(best_v[col * TPC + sgm], best_i[col * TPC + sgm], x, ix)) { x = best_v[col * TPC + sgm]; ix = best_i[col * TPC + sgm]; }
          p.am_val[(size_t)m * gridDim.x + tile_a] = x;
          p.am_idx[(size_t)m * gridDim.x + tile_a] = ix;
        }
      }
    }
  }
  if (p.splits > 1 || p.swiglu || p.rope) {
    // split K: every thread of every CTA of the cluster passes both cluster barriers; only the epilogue warps work
    // between them. Without a split (fused SwiGLU only) the epilogue warps synchronise among themselves.
    if (p.splits > 1) cluster_sync_all();
    if (warp >= 2) {
      if (p.splits == 1) asm volatile("bar.sync 1, 128;" ::: "memory");
      const int r = (warp & 3) * 32 + lane;
      const int feat = tile_a * BM + r;
      const uint32_t rank = p.splits > 1 ? cluster_rank() : 0u;
      const int cols = min(BN, p.rows - tile_b * BN);
      const float bv = (p.bias && feat < p.feats) ? p.bias[feat] : 0.f;
      const uint32_t base = smem_u32(smem) + (uint32_t)r * 4u;
      float* ex = (float*)smem + BN * BM;            // [16][128]: a group of columns, for the gate / up exchange
      int n_my = cols > (int)rank ? (cols - (int)rank + p.splits - 1) / p.splits : 0;   // columns rank, rank + S, ...
      if (p.swiglu && p.splits == 1) {
        // K not split: the tile is complete in this CTA's shared memory as [token][feature]. Thread r and thread r + 64
        // share feature r of the tile's 64 (gate in row r, up in row r + 64) and take every other token; the loop is
        // unrolled so that the loads, exponentials and divisions of eight tokens are in flight together (two of the
        // four warps walking the tokens one by one took 14 us of a 58 us product at 64 tokens).
        const int f = r & 63, par = r >> 6, gate_feat = tile_a * BM + f;
        if (gate_feat < p.feats) {
          const float bg = p.bias ? p.bias[gate_feat] : 0.f, bu = p.bias ? p.bias[gate_feat + 64] : 0.f;
          const float* tile = (const float*)smem;
          __nv_bfloat16* dst = p.c_bf16 + (size_t)(tile_b * BN) * (p.feats >> 1) + tile_a * 64 + f;
#pragma unroll 8
          for (int c = par; c < cols; c += 2)
            dst[(size_t)c * (p.feats >> 1)] = __float2bfloat16_rn(silu_mul(tile[c * BM + f] + bg, tile[c * BM + f + 64] + bu));
        }
        n_my = 0;
      }
      if (p.splits > 1 && !p.swiglu && !p.rope) {
        // the plain sum over the splits: four columns' partial results asked for before the first is added up
#pragma unroll 4
        for (int i = 0; i < n_my; ++i) {
          const int c = (int)rank + i * p.splits;
          float v[8];
#pragma unroll
          for (int sp = 0; sp < 8; ++sp) v[sp] = sp < p.splits ? ld_dsmem(base + (uint32_t)(c * BM) * 4u, (uint32_t)sp) : 0.f;
          float acc = 0.f;
#pragma unroll
          for (int sp = 0; sp < 8; ++sp) acc += v[sp];
          if (feat < p.feats) {
            const int m = tile_b * BN + c;
            if (p.c_f32) p.c_f32[(size_t)m * p.feats + feat] = acc + bv;
            else p.c_bf16[(size_t)m * p.feats + feat] = __float2bfloat16_rn(acc + bv);
          }
        }
        n_my = 0;
      }
      for (int i0 = 0; i0 < n_my; i0 += 16) {
        const int ni = min(16, n_my - i0);
#pragma unroll 2
        for (int i = 0; i < ni; ++i) {
          const int c = (int)rank + (i0 + i) * p.splits;
          float acc = 0.f;
          if (p.splits > 1) {
            // all splits' partials are asked for before the first is used (a cluster holds at most 8 CTAs); the sum
            // runs in split order
            float v[8];
#pragma unroll
            for (int sp = 0; sp < 8; ++sp) v[sp] = sp < p.splits ? ld_dsmem(base + (uint32_t)(c * BM) * 4u, (uint32_t)sp) : 0.f;
#pragma unroll
            for (int sp = 0; sp < 8; ++sp) acc += v[sp];
          } else {
            acc = ((const float*)smem)[c * BM + r];
          }
          const float y = acc + bv;
          if (p.swiglu || p.rope) {
            ex[i * BM + r] = y;
          } else if (feat < p.feats) {
            const int m = tile_b * BN + c;
            if (p.c_f32) p.c_f32[(size_t)m * p.feats + feat] = y;
            else p.c_bf16[(size_t)m * p.feats + feat] = __float2bfloat16_rn(y);
          }
        }
        if (p.swiglu) {
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (r < 64) {
            const int half = p.feats >> 1;
            for (int i = 0; i < ni; ++i) {
              const int m = tile_b * BN + (int)rank + (i0 + i) * p.splits;
              p.c_bf16[(size_t)m * half + tile_a * 64 + r] = __float2bfloat16_rn(silu_mul(ex[i * BM + r], ex[i * BM + r + 64]));
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        if (p.rope) {
          asm volatile("bar.sync 1, 128;" ::: "memory");
          const int hd = p.hd, half = hd >> 1;
          const int head = feat / hd, j = feat - head * hd;      // (a tile starts at a head's first feature: hd divides 128)
          if (feat < p.feats) {
            for (int i = 0; i < ni; ++i) {
              const int m = tile_b * BN + (int)rank + (i0 + i) * p.splits;
              // (columns 0 .. PRE - 1 of this thread were looked up at the kernel's start; i0 is 0 for them)
              const bool ahead = i0 + i < PRE;
              int row = 0, ps = 0, page_ahead = -1;
              float cs = 0.f, sn = 0.f;
#pragma unroll
              for (int q = 0; q < PRE; ++q)
                if (i0 + i == q) { row = pre_row[q]; ps = pre_ps[q]; page_ahead = pre_page[q]; cs = pre_cos[q]; sn = pre_sin[q]; }
              if (!ahead) { row = p.seq_row[m]; ps = p.pos[m]; }
              const bool in_range = ps >= 0 && ps < p.max_len;
              if (row >= 0 && !in_range && r == 0) atomicOr(p.err, FZ_ERR_POS_RANGE);
              const bool live = row >= 0 && in_range;
              __nv_bfloat16* dst = nullptr;
              if (head < p.Hq) {
                dst = p.c_bf16 + ((size_t)m * p.Hq + head) * hd;
              } else if (live && p.write) {
                const int page = ahead ? page_ahead : p.table[(size_t)row * p.mb + ps / p.page_size];
                if (page < 0) {
                  if (j == 0 && head == p.Hq) atomicOr(p.err, FZ_ERR_NO_PAGE);
                } else {
                  const long long slot = (long long)page * p.page_stride + (long long)(ps % p.page_size) * hd;
                  const long long head_stride = (long long)p.page_size * hd;
                  dst = head < p.Hq + p.Hkv ? p.k_pool + slot + (long long)(head - p.Hq) * head_stride
                                            : p.v_pool + slot + (long long)(head - p.Hq - p.Hkv) * head_stride;
                }
              }
              if (dst == nullptr) continue;
              if (head >= p.Hq + p.Hkv) {
                dst[j] = __float2bfloat16_rn(ex[i * BM + r]);
              } else if (j < half) {
                float o1 = 0.f, o2 = 0.f;
                if (live && !ahead) { cs = p.cos_t[(size_t)ps * half + j]; sn = p.sin_t[(size_t)ps * half + j]; }
                if (live) fz_rope_pair(ex[i * BM + r], ex[i * BM + r + half], cs, sn, o1, o2);
                dst[j] = __float2bfloat16_rn(o1);
                dst[j + half] = __float2bfloat16_rn(o2);
              }
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
      }
    }
    if (p.splits > 1) cluster_sync_all();    // nobody leaves while its shared memory may still be read
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_d, TMEM_COLS);
  }
  if (threadIdx.x == 0 && flag[1]) atomicOr(p.err, FZ_ERR_WAIT_TIMEOUT);
}

// Rows mode: one thread's lane (token row `row`) of a finished accumulator of BN columns at `taddr`, with the bias added,
// to the output's columns n0 .. n0 + BN - 1 (or, with the fused SwiGLU, to its packed half). Every lane of the warp takes
// part in the loads from tensor memory whether or not its row exists.
template <int BN>
__device__ __forceinline__ void rows_store_tile(const Params& p, uint32_t taddr, int row, int n0) {
  float v[16];
  if (p.swiglu) {
    // columns [128 b, 128 b + 64) are gate, [128 b + 64, 128 b + 128) up of output features 64 (n0 / 128 + b) ..
    float u[16];
#pragma unroll 1
    for (int c = 0; c < BN; c += 16) {
      if ((c & 64) != 0) continue;
      tmem_ld16(taddr + (uint32_t)c, v);
      tmem_ld16(taddr + (uint32_t)(c + 64), u);
      const int n = n0 + c;                       // packed index of the gate column
      if (row >= p.rows || n >= p.feats) continue;
      uint32_t w[8];
#pragma unroll
      for (int i = 0; i < 16; i += 2) {
        const float g0 = v[i] + (p.bias ? p.bias[n + i] : 0.f), g1 = v[i + 1] + (p.bias ? p.bias[n + i + 1] : 0.f);
        const float u0 = u[i] + (p.bias ? p.bias[n + 64 + i] : 0.f), u1 = u[i + 1] + (p.bias ? p.bias[n + 64 + i + 1] : 0.f);
        const __nv_bfloat162 h2 = __floats2bfloat162_rn(silu_mul(g0, u0), silu_mul(g1, u1));
        w[i >> 1] = *(const uint32_t*)&h2;
      }
      uint4* dst = (uint4*)(p.c_bf16 + (size_t)row * (p.feats >> 1) + (n >> 7) * 64 + (n & 63));
      dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
      dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
    }
    return;
  }
#pragma unroll 1
  for (int c = 0; c < BN; c += 16) {
    tmem_ld16(taddr + (uint32_t)c, v);
    if (row >= p.rows) continue;
    const int n = n0 + c;
    if (p.vec_ok && n + 16 <= p.feats) {
      if (p.bias) {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] += p.bias[n + i];
      }
      if (p.c_f32) {
        float4* dst = (float4*)(p.c_f32 + (size_t)row * p.feats + n);
#pragma unroll
        for (int i = 0; i < 4; ++i) dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
      } else {
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const __nv_bfloat162 h2 = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
          w[i] = *(const uint32_t*)&h2;
        }
        uint4* dst = (uint4*)(p.c_bf16 + (size_t)row * p.feats + n);
        dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
        dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        if (n + i < p.feats) {
          const float y = v[i] + (p.bias ? p.bias[n + i] : 0.f);
          if (p.c_f32) p.c_f32[(size_t)row * p.feats + n + i] = y;
          else p.c_bf16[(size_t)row * p.feats + n + i] = __float2bfloat16_rn(y);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------- rows mode, persistent
// C[rows, feats] = X . W^T (+ bias) for many token rows. grid = min(tiles, SMs); tile i of a CTA is tile number
// blockIdx.x + i * gridDim.x, token tile = number % tiles_m, feature tile = number / tiles_m.
template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_rows_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const Params p,
                    int tiles_m, int tiles_n) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = 2 * BN <= 32 ? 32 : 2 * BN <= 64 ? 64 : 2 * BN <= 128 ? 128 : 2 * BN <= 256 ? 256 : 512;   // two accumulators (a power of two)
  uint64_t* full = (uint64_t*)(smem + (size_t)p.stages * STAGE_BYTES);
  uint64_t* empty = full + p.stages;
  uint64_t* acc_full = empty + p.stages;     // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2]
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  int* flag = (int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kblocks = (p.K + BK - 1) / BK;
  const int total = tiles_m * tiles_n;
  const int my_tiles = total > (int)blockIdx.x ? (total - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 128); }
    flag[0] = 0;
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  fz_grid_launch_dependents();
  if (warp != 0) fz_grid_wait();

  if (warp == 0) {
    if (lane == 0) {
      // weights of the first stages before the wait on the previous kernel (they do not depend on it)
      const int first = (int)blockIdx.x;
      const int early = my_tiles > 0 ? (kblocks < p.stages ? kblocks : p.stages) : 0;
      for (int i = 0; i < early; ++i) {
        mbar_expect_tx(&full[i], STAGE_BYTES);
        tma_load_2d(smem + (size_t)i * STAGE_BYTES + A_BYTES, &map_w, &full[i], i * BK, (first / tiles_m) * BN);
      }
      fz_grid_wait();
      // (the stage and its round are kept by counting: this one lane feeds the whole pipeline, and a division per
      // k-block would make it the slowest part)
      int it = 0, s = 0, round = 0;
      bool ok = true;
      for (int j = 0; j < my_tiles && ok; ++j) {
        const int tile = (int)blockIdx.x + j * (int)gridDim.x;
        const int tm = tile % tiles_m, tn = tile / tiles_m;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          uint8_t* sa = smem + (size_t)s * STAGE_BYTES;
          if (it >= early) {
            if (round > 0 && !mbar_wait(&empty[s], (round - 1) & 1)) { flag[0] = 1; ok = false; break; }
            mbar_expect_tx(&full[s], STAGE_BYTES);
            tma_load_2d(sa + A_BYTES, &map_w, &full[s], kb * BK, tn * BN);
          }
          tma_load_2d(sa, &map_x, &full[s], kb * BK, tm * BM);
          if (++s == p.stages) { s = 0; ++round; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN);
      int s = 0, round = 0;
      bool ok = true;
      for (int j = 0; j < my_tiles && ok; ++j) {
        const int acc = j & 1;
        if (j >= 2 && !mbar_wait(&acc_empty[acc], ((j >> 1) - 1) & 1)) { flag[0] = 1; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&full[s], round & 1)) { flag[0] = 1; ok = false; break; }
          tc_fence_after();
          const uint8_t* sa = smem + (size_t)s * STAGE_BYTES;
          const uint64_t da = desc_k_major(smem_u32(sa)), db = desc_k_major(smem_u32(sa + A_BYTES));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16(tmem_d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty[s]);
          if (++s == p.stages) { s = 0; ++round; }
        }
        umma_commit(&acc_full[acc]);
      }
    }
  } else {
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    bool ok = true;
    for (int j = 0; j < my_tiles && ok; ++j) {
      const int tile = (int)blockIdx.x + j * (int)gridDim.x;
      const int tm = tile % tiles_m, tn = tile / tiles_m;
      const int acc = j & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&acc_full[acc], (j >> 1) & 1));
      if (!ok) { flag[0] = 1; break; }
      tc_fence_after();
      // (Four epilogue warps here. Eight, as in the two-SM kernel, were measured on this kernel and did not pay: the tiles
      // it gets are narrow or few, and 2,048 tokens at Qwen2.5-0.5B sizes took 3.94 ms with them against 3.77 ms.)
      const uint32_t taddr = tmem_base + (uint32_t)(acc * BN) + ((uint32_t)(quad * 32) << 16);
      rows_store_tile<BN>(p, taddr, tm * BM + r, tn * BN);
      tc_fence_before();
      mbar_arrive(&acc_empty[acc]);      // this thread has read its lane of the accumulator
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && flag[0]) atomicOr(p.err, FZ_ERR_WAIT_TIMEOUT);
}

template <int BN>
int launch_rows(const CUtensorMap& mx, const CUtensorMap& mw, const Params& p, int tiles_m, int tiles_n, cudaStream_t stream) {
  constexpr int STAGE_BYTES = (BM + BN) * BK * 2;
  const size_t smem = (size_t)p.stages * STAGE_BYTES + 1024 + 8 * (2 * p.stages + 4) + 16;
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_rows_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    allowed = smem;
  }
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  const int total = tiles_m * tiles_n;
  dim3 grid(total < sms ? total : sms);
  fz_launch(gemm_tc_rows_kernel<BN>, grid, dim3(NUM_THREADS), smem, stream, mx, mw, p, tiles_m, tiles_n);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

// ---------------------------------------------------------------------------------------------- rows mode, two SMs per tile
// The same product with a pair of CTAs (a cluster of two, on the two SMs of one TPC) on every 256 x 256 output tile:
// `tcgen05.mma.cta_group::2` multiplies 256 token rows by 256 features per instruction, each CTA holding its 128 token
// rows of X and its 128 of the 256 features of W in its own shared memory, and its 128 rows of the accumulator in its own
// tensor memory. Per SM and k-block that is 32 KB of operands instead of 48 KB for the same 128 x 256 outputs: less L2
// and shared-memory traffic, more stages in the ring, half as many instructions to issue.
//
// Who signals whom: each CTA's producer lane loads its own two operand tiles (`cp.async.bulk.tensor ... .cta_group::2`,
// which may count its bytes on the other CTA's barrier; no multicast) and has them counted on the `full` barrier of the
// leader (cluster rank 0), whose producer expects both CTAs' bytes. The leader's MMA lane issues the instructions for
// the pair and commits them to the `empty` (and, per tile, `acc_full`) barriers of BOTH CTAs (`tcgen05.commit` with a CTA
// mask), so each producer refills its own ring and each CTA's epilogue warps read their own tensor memory. One lane of
// each epilogue warp of both CTAs then arrives on the leader's `acc_empty` barrier (count 16). Every wait is bounded;
// both CTAs pass a cluster barrier after the barriers' initialisation and before they leave.
constexpr int PAIR_BN = 256;

__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
  return remote;
}
__device__ __forceinline__ uint32_t ld_dsmem_u32(uint32_t cluster_addr) {
  uint32_t v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(cluster_addr) : "memory");
  return v;
}
// A tile into this CTA's shared memory, its bytes counted on a barrier given by its cluster address (this CTA's or its
// pair's).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y) : "memory");
}
// D (256 rows over the pair's tensor memories) (+)= A (each CTA's 128 rows) * B (each CTA's half of the N columns)
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on the barrier at this shared-memory offset in both CTAs of the pair (cluster ranks `first` and `first` + 1) when
// the MMAs issued so far are complete.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint32_t first = 0u) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((uint16_t)(3u << first)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

// Tensor memory for a pair: allocated for the pair as one (`cta_group::2`, executed by a warp of each CTA), so that both
// CTAs hold the same columns whatever else is resident on their SMs (measured with two CTAs per SM: separate
// `cta_group::1` allocations gave the CTAs of a pair different columns, this gives them the same); the kernels still
// compare the two addresses before they compute anything.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}

__global__ void __launch_bounds__(PAIR_THREADS_G, 1)
gemm_tc_rows_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const Params p,
                         int tiles_m, int tiles_n) {
  constexpr int BN = PAIR_BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int A_BYTES = BM * BK * 2, B_BYTES = (BN / 2) * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = 2 * BN;          // two accumulators of 256 columns
  uint64_t* full = (uint64_t*)(smem + (size_t)p.stages * STAGE_BYTES);      // used in the leader only
  uint64_t* empty = full + p.stages;
  uint64_t* acc_full = empty + p.stages;     // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2], used in the leader only
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  int* flag = (int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();      // 0: the leader
  const int pair = (int)blockIdx.x >> 1, pairs = (int)gridDim.x >> 1;
  const int kblocks = (p.K + BK - 1) / BK;
  const int total = tiles_m * tiles_n;
  const int my_tiles = total > pair ? (total - pair + pairs - 1) / pairs : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 16); }
    flag[0] = 0;
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();      // the pair's barriers exist and its tensor memory is allocated before anything crosses over
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // One instruction writes the same tensor-memory address in both CTAs: the pair's allocation gives both the same
  // columns; if the two addresses ever differed, nothing is computed and the error is reported.
  const bool same_base = ld_dsmem_u32(map_to_cta(smem_u32(tmem_slot), rank ^ 1u)) == tmem_base;
  fz_grid_launch_dependents();
  if (warp != 0) fz_grid_wait();

  if (!same_base) {
    if (threadIdx.x == 0) flag[0] = 1;
  } else if (warp == 0) {
    if (lane == 0) {
      const uint32_t full0 = map_to_cta(smem_u32(full), 0u);      // the leader's `full` barriers, 8 bytes apart
      const uint32_t s0 = smem_u32(smem);
      // weights of the first stages before the wait on the previous kernel (they do not depend on it)
      const int first = pair;
      const int early = my_tiles > 0 ? (kblocks < p.stages ? kblocks : p.stages) : 0;
      for (int i = 0; i < early; ++i) {
        if (rank == 0) mbar_expect_tx(&full[i], 2 * STAGE_BYTES);
        tma_load_2d_pair(s0 + (uint32_t)(i * STAGE_BYTES + A_BYTES), &map_w, full0 + 8u * (uint32_t)i, i * BK,
                         (first / tiles_m) * BN + (int)rank * (BN / 2));
      }
      fz_grid_wait();
      int it = 0, s = 0, round = 0;
      bool ok = true;
      for (int j = 0; j < my_tiles && ok; ++j) {
        const int tile = pair + j * pairs;
        const int tm = tile % tiles_m, tn = tile / tiles_m;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t sa = s0 + (uint32_t)(s * STAGE_BYTES);
          if (it >= early) {
            if (round > 0 && !mbar_wait(&empty[s], (round - 1) & 1)) { flag[0] = 1; ok = false; break; }
            if (rank == 0) mbar_expect_tx(&full[s], 2 * STAGE_BYTES);
            tma_load_2d_pair(sa + A_BYTES, &map_w, full0 + 8u * (uint32_t)s, kb * BK, tn * BN + (int)rank * (BN / 2));
          }
          tma_load_2d_pair(sa, &map_x, full0 + 8u * (uint32_t)s, kb * BK, (2 * tm + (int)rank) * BM);
          if (++s == p.stages) { s = 0; ++round; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc(2 * BM, BN);
      int s = 0, round = 0;
      bool ok = true;
      for (int j = 0; j < my_tiles && ok; ++j) {
        const int acc = j & 1;
        if (j >= 2 && !mbar_wait(&acc_empty[acc], ((j >> 1) - 1) & 1)) { flag[0] = 1; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&full[s], round & 1)) { flag[0] = 1; ok = false; break; }
          tc_fence_after();
          const uint8_t* sa = smem + (size_t)s * STAGE_BYTES;
          const uint64_t da = desc_k_major(smem_u32(sa)), db = desc_k_major(smem_u32(sa + A_BYTES));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16_pair(tmem_d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(&empty[s]);
          if (++s == p.stages) { s = 0; ++round; }
        }
        umma_commit_pair(&acc_full[acc]);
      }
    }
  } else {
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t acc_empty0 = map_to_cta(smem_u32(acc_empty), 0u);
    bool ok = true;
    for (int j = 0; j < my_tiles && ok; ++j) {
      const int tile = pair + j * pairs;
      const int tm = tile % tiles_m, tn = tile / tiles_m;
      const int acc = j & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&acc_full[acc], (j >> 1) & 1));
      if (!ok) { flag[0] = 1; break; }
      tc_fence_after();
      // (warps 2..5 take the tile's first 128 columns, warps 6..9 the other 128: two warps per scheduler, so that one
      // computes while the other waits; with four warps the epilogue of a tile took longer than the products of a tile
      // with a short K: 13 us per tile at K = 896, where the products take 5)
      const int col0 = warp >= 6 ? BN / 2 : 0;
      const uint32_t taddr = tmem_base + (uint32_t)(acc * BN + col0) + ((uint32_t)(quad * 32) << 16);
      rows_store_tile<BN / 2>(p, taddr, (2 * tm + (int)rank) * BM + r, tn * BN + col0);
      tc_fence_before();
      __syncwarp();      // every lane of the warp has read its lane of the accumulator
      if (lane == 0) mbar_arrive_cluster(acc_empty0 + 8u * (uint32_t)acc);
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();      // nobody leaves while the other CTA may still signal its barriers or write its tensor memory
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && flag[0]) atomicOr(p.err, FZ_ERR_WAIT_TIMEOUT);
}

int launch_rows_pair(const CUtensorMap& mx, const CUtensorMap& mw, const Params& p, int tiles_m, int tiles_n, int sms, cudaStream_t stream) {
  constexpr int STAGE_BYTES = (BM + PAIR_BN / 2) * BK * 2;
  const size_t smem = (size_t)p.stages * STAGE_BYTES + 1024 + 8 * (2 * p.stages + 4) + 16;
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_rows_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    allowed = smem;
  }
  const int total = tiles_m * tiles_n, most = sms / 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * (unsigned)(total < most ? total : most));
  cfg.blockDim = dim3(PAIR_THREADS_G);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (fz_pdl_enabled()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  attr[na].id = cudaLaunchAttributeClusterDimension;
  attr[na].val.clusterDim.x = 2;
  attr[na].val.clusterDim.y = 1;
  attr[na].val.clusterDim.z = 1;
  ++na;
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t le = cudaLaunchKernelEx(&cfg, gemm_tc_rows_pair_kernel, mx, mw, p, tiles_m, tiles_n);
  if (le != cudaSuccess) return (int)le;
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

// ---------------------------------------------------------------------------------------------- rows mode, K split
// C[rows, feats] = X . W^T (+ bias) for a few hundred token rows, where the 128 x 256 output tiles are far fewer than the
// SMs: a tile's range of K is cut into `splits` pieces, one CTA each, and the CTAs of a tile form a thread-block cluster.
// A CTA can draw operands from L2 / HBM only at the rate its shared-memory ring and the memory latency allow (about
// 90 GB/s), so a tile that walks a long K alone takes its bytes / that rate, whatever the tensor core could do; cut in
// pieces, more SMs draw at once. Every CTA leaves its float32 partial tile in its own shared memory (row-major, rows
// padded by four floats so that neither the writes nor the reads collide on the banks); after a cluster barrier CTA r
// adds, for its share of the tile's columns, the partials of all splits in split order through distributed shared
// memory, adds the bias and stores. No partial goes to global memory; the sum has one fixed order.
constexpr int SPLIT_BN = 256;
constexpr int SPLIT_LD = SPLIT_BN + 4;      // floats per row of the partial tile

__device__ __forceinline__ float4 ld_dsmem_v4(uint32_t addr, uint32_t rank) {
  uint32_t remote;
  float4 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote));
  return v;
}

// The reduction of the K-cut many-token kernel for one token row: the column groups g0 .. g1 - 1 (four columns each) of
// the tile, every group the sum over the S splits' partial tiles in split order (read through distributed shared
// memory; U groups' loads are in flight together), plus the bias, stored.
template <bool PAIR, int S, int U>
__device__ __forceinline__ void split_reduce_rows(const Params& p, uint32_t base, int g0, int g1, int n0, int row, uint32_t half) {
  for (int gb = g0; gb < g1; gb += U) {
    float4 v[U][S];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int sp = 0; sp < S; ++sp)      // the CTA of split sp that holds the same rows: cluster rank sp, or 2 sp + half
        v[u][sp] = gb + u < g1 ? ld_dsmem_v4(base + (uint32_t)(4 * (gb + u)) * 4u, PAIR ? 2u * (uint32_t)sp + half : (uint32_t)sp)
                               : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int g = gb + u;
      if (g >= g1) break;
      const int n = n0 + 4 * g;
      if (n >= p.feats) break;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int sp = 0; sp < S; ++sp) { acc.x += v[u][sp].x; acc.y += v[u][sp].y; acc.z += v[u][sp].z; acc.w += v[u][sp].w; }
      float y[4] = {acc.x, acc.y, acc.z, acc.w};
      if (p.vec_ok && n + 4 <= p.feats) {
        if (p.bias) {
#pragma unroll
          for (int j = 0; j < 4; ++j) y[j] += p.bias[n + j];
        }
        if (p.c_f32) {
          *(float4*)(p.c_f32 + (size_t)row * p.feats + n) = make_float4(y[0], y[1], y[2], y[3]);
        } else {
          const __nv_bfloat162 lo = __floats2bfloat162_rn(y[0], y[1]), hi = __floats2bfloat162_rn(y[2], y[3]);
          *(uint2*)(p.c_bf16 + (size_t)row * p.feats + n) = make_uint2(*(const uint32_t*)&lo, *(const uint32_t*)&hi);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (n + j < p.feats) {
            const float yj = y[j] + (p.bias ? p.bias[n + j] : 0.f);
            if (p.c_f32) p.c_f32[(size_t)row * p.feats + n + j] = yj;
            else p.c_bf16[(size_t)row * p.feats + n + j] = __float2bfloat16_rn(yj);
          }
        }
      }
    }
  }
}

// PAIR: the tile is 256 token rows by 256 features on a pair of CTAs (`tcgen05.mma.cta_group::2`, as in
// `gemm_tc_rows_pair_kernel`: each CTA loads its 128 rows of X and 128 of the 256 features of W, so a CTA draws 32 KB per
// k-block instead of 48 KB), the cluster is (2, 1, splits) with the two CTAs of a pair at neighbouring ranks, and a CTA
// adds up the partial tiles of its own half of the rows.
template <bool PAIR>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_rows_split_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const Params p) {
  constexpr int BN = SPLIT_BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int A_BYTES = BM * BK * 2, B_BYTES = (PAIR ? BN / 2 : BN) * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  uint64_t* full = (uint64_t*)(smem + (size_t)p.stages * STAGE_BYTES);      // PAIR: used in the pair's leader only
  uint64_t* empty = full + p.stages;
  uint64_t* acc_ready = empty + p.stages;
  uint32_t* tmem_slot = (uint32_t*)(acc_ready + 1);
  int* flag = (int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const uint32_t half = PAIR ? (rank & 1u) : 0u, leader = PAIR ? (rank & ~1u) : rank;      // which rows of the pair's tile; its first CTA
  const int tm = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x, tn = blockIdx.y, split = blockIdx.z;
  const int row0 = PAIR ? (2 * tm + (int)half) * BM : tm * BM;
  const int w_row0 = tn * BN + (PAIR ? (int)half * (BN / 2) : 0);
  const int kblocks = (p.K + BK - 1) / BK;
  const int kb0 = (int)((long long)kblocks * split / p.splits), kb1 = (int)((long long)kblocks * (split + 1) / p.splits);
  const int nkb = kb1 - kb0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(acc_ready, 1);
    flag[0] = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    if constexpr (PAIR) tmem_alloc_pair(tmem_slot, BN); else tmem_alloc(tmem_slot, BN);
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();      // the pair's barriers and tensor memory exist before anything crosses over
  tc_fence_after();
  const uint32_t tmem_d = *tmem_slot;
  bool same_base = true;      // (one instruction writes the same tensor-memory address in both CTAs of a pair)
  if constexpr (PAIR) same_base = ld_dsmem_u32(map_to_cta(smem_u32(tmem_slot), rank ^ 1u)) == tmem_d;
  fz_grid_launch_dependents();
  if (warp != 0) fz_grid_wait();

  if (!same_base) {
    if (threadIdx.x == 0) flag[0] = 1;
  } else if (warp == 0) {
    if (lane == 0) {
      const uint32_t s0 = smem_u32(smem);
      const uint32_t full0 = PAIR ? map_to_cta(smem_u32(full), leader) : smem_u32(full);      // barriers are 8 bytes apart
      const uint32_t expect = PAIR ? 2 * STAGE_BYTES : STAGE_BYTES;
      auto load = [&](uint32_t dst, const CUtensorMap* map, int stage, int x, int y) {
        if constexpr (PAIR) tma_load_2d_pair(dst, map, full0 + 8u * (uint32_t)stage, x, y);
        else tma_load_2d_u32(dst, map, full0 + 8u * (uint32_t)stage, x, y);
      };
      // the weights of the first stages before the wait on the previous kernel (they do not depend on it)
      const int early = nkb < p.stages ? nkb : p.stages;
      for (int i = 0; i < early; ++i) {
        if (half == 0) mbar_expect_tx(&full[i], expect);
        load(s0 + (uint32_t)(i * STAGE_BYTES + A_BYTES), &map_w, i, (kb0 + i) * BK, w_row0);
      }
      fz_grid_wait();
      for (int i = 0, s = 0, round = 0; i < nkb; ++i) {
        const uint32_t sa = s0 + (uint32_t)(s * STAGE_BYTES);
        if (round > 0) {
          if (!mbar_wait(&empty[s], (round - 1) & 1)) { flag[0] = 1; break; }
          if (half == 0) mbar_expect_tx(&full[s], expect);
          load(sa + A_BYTES, &map_w, s, (kb0 + i) * BK, w_row0);
        }
        load(sa, &map_x, s, (kb0 + i) * BK, row0);
        if (++s == p.stages) { s = 0; ++round; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && half == 0) {
      constexpr uint32_t idesc = make_idesc(PAIR ? 2 * BM : BM, BN);
      for (int i = 0, s = 0, round = 0; i < nkb; ++i) {
        if (!mbar_wait(&full[s], round & 1)) { flag[0] = 1; break; }
        tc_fence_after();
        const uint8_t* sa = smem + (size_t)s * STAGE_BYTES;
        const uint64_t da = desc_k_major(smem_u32(sa)), db = desc_k_major(smem_u32(sa + A_BYTES));
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          if constexpr (PAIR) umma_bf16_pair(tmem_d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (i > 0 || k > 0) ? 1u : 0u);
          else umma_bf16(tmem_d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (i > 0 || k > 0) ? 1u : 0u);
        }
        if constexpr (PAIR) umma_commit_pair(&empty[s], leader); else umma_commit(&empty[s]);
        if (++s == p.stages) { s = 0; ++round; }
      }
      if constexpr (PAIR) umma_commit_pair(acc_ready, leader); else umma_commit(acc_ready);
    }
  } else {
    // the accumulator -> this CTA's partial tile in shared memory (every stage has been consumed by now, in both CTAs
    // of a pair: the commit covers the pair's instructions, which read both)
    const int quad = warp & 3, r = quad * 32 + lane;
    const bool ok = __all_sync(0xffffffffu, mbar_wait(acc_ready, 0));
    if (!ok) flag[0] = 1;
    tc_fence_after();
    const uint32_t taddr = tmem_d + ((uint32_t)(quad * 32) << 16);
    float* part = (float*)smem + (size_t)r * SPLIT_LD;
    float v[16];
#pragma unroll 1
    for (int c = 0; c < BN; c += 16) {
      if (ok && nkb > 0) tmem_ld16(taddr + (uint32_t)c, v);
      else {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < 16; j += 4) *(float4*)(part + c + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    }
  }
  // every thread of every CTA of the cluster passes both cluster barriers; only the epilogue warps work between them
  cluster_sync_all();
  if (warp >= 2 && same_base) {
    const int r = (warp & 3) * 32 + lane;
    const int row = row0 + r;
    // this CTA's share of the tile's columns, in groups of four
    const int groups = BN / 4;
    const int g0 = (int)((long long)groups * split / p.splits), g1 = (int)((long long)groups * (split + 1) / p.splits);
    const uint32_t base = smem_u32(smem) + (uint32_t)r * (uint32_t)(SPLIT_LD * 4);
    if (row < p.rows) {
      // (with two splits a thread has 32 groups: eight groups' partial tiles are asked for at once, which took 1 to 2 us
      // off products of 28 to 61 us; with four splits and 16 groups the same was measured and lost a little)
      if (p.splits == 2) split_reduce_rows<PAIR, 2, 8>(p, base, g0, g1, tn * BN, row, half);
      else if (p.splits == 4) split_reduce_rows<PAIR, 4, 2>(p, base, g0, g1, tn * BN, row, half);
      else split_reduce_rows<PAIR, 8, 2>(p, base, g0, g1, tn * BN, row, half);
    }
  }
  cluster_sync_all();      // nobody leaves while its shared memory may still be read
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    if constexpr (PAIR) tmem_dealloc_pair(tmem_d, BN); else tmem_dealloc(tmem_d, BN);
  }
  if (threadIdx.x == 0 && flag[0]) atomicOr(p.err, FZ_ERR_WAIT_TIMEOUT);
}

template <bool PAIR>
int launch_rows_split(const CUtensorMap& mx, const CUtensorMap& mw, const Params& p, int tiles_m, int tiles_n, cudaStream_t stream) {
  constexpr int STAGE_BYTES = (BM + (PAIR ? SPLIT_BN / 2 : SPLIT_BN)) * BK * 2;
  const size_t ring = (size_t)p.stages * STAGE_BYTES, partial = (size_t)BM * SPLIT_LD * 4;
  const size_t smem = (ring > partial ? ring : partial) + 1024 + 8 * (2 * p.stages + 1) + 16;
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_rows_split_kernel<PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    allowed = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((PAIR ? 2 : 1) * tiles_m, tiles_n, p.splits);      // PAIR: tiles_m counts tiles of 256 rows
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (fz_pdl_enabled()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  attr[na].id = cudaLaunchAttributeClusterDimension;
  attr[na].val.clusterDim.x = PAIR ? 2 : 1;
  attr[na].val.clusterDim.y = 1;
  attr[na].val.clusterDim.z = (unsigned)p.splits;
  ++na;
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t le = cudaLaunchKernelEx(&cfg, gemm_tc_rows_split_kernel<PAIR>, mx, mw, p);
  if (le != cudaSuccess) return (int)le;
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

// ---------------------------------------------------------------------------------------------- host side
template <int BN>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const Params& p, dim3 grid, cudaStream_t stream) {
  constexpr int STAGE_BYTES = (BM + BN) * BK * 2;
  const size_t smem = (size_t)p.stages * STAGE_BYTES + 1024 + 8 * (2 * p.stages + 1) + 16;
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    allowed = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (fz_pdl_enabled()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (p.splits > 1) {      // the splits of one tile are one cluster (z dimension)
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = (unsigned)p.splits;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t le = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN>, ma, mb, p);
  if (le != cudaSuccess) return (int)le;
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

int pick_stages(int bn) {
  const int stage = (BM + bn) * BK * 2;
  int s = (200 * 1024) / stage;
  if (bn <= 128) s = (100 * 1024) / stage;  // few-token mode: leaves room for two CTAs per SM
  return s < 2 ? 2 : (s > 8 ? 8 : s);
}
}  // namespace

// Can this kernel take the product? K a multiple of 8 (16-byte rows for TMA), operands 16-byte aligned.
FZ_API int fz_gemm_tc_check(const void* x, const void* w, int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0) return FZ_BAD_SHAPE;
  if (K % 8) return FZ_BAD_SHAPE;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return FZ_BAD_ALIGNMENT;
  return FZ_OK;
}

// The number of K splits for a product with these N and K in swap mode: from N and K only, so that a token row's sum
// order never depends on how many rows share the step.
FZ_API int fz_gemm_tc_splits(int N, int K) {
  const int tiles = (N + BM - 1) / BM, kblocks = (K + BK - 1) / BK;
  // Two CTAs fit each of the 148 SMs, but clusters do not pack the GPCs perfectly: measured on B200, 48 clusters of 6
  // (288 CTAs) need a second wave (19 us for the 6144 x 4096 product) where 48 of 5 (13 us) and 32 of 8 do not. So the
  // CTA count stays at or below 256.
  // (Down to one k-block of 64 per piece: small products are bound by the chain of a single CTA's loads and
  // instructions, not by bytes, and more pieces shorten it. Measured at Qwen2.5-0.5B sizes, batch 8, two engines
  // alternating in one process: at least 4 k-blocks per piece 1.040 ms per step, 3: 0.992, 2: 0.956, 1: 0.936.)
  int s = 256 / tiles;
  if (s > kblocks) s = kblocks;
  if (s > 8) s = 8;                  // a portable cluster holds at most 8 CTAs
  return s < 1 ? 1 : s;
}

// The number of K pieces a product of M > 128 token rows is cut into (1: not cut): only where the 128 x 256 tiles are at
// most half as many as the SMs, no piece shorter than 8 k-blocks of 64, and a power of two: with one CTA per SM, clusters
// of three do not pack the GPCs (measured: 48 clusters of 3 need a second wave, 45 us for the 256 x 6144 x 4096 product
// where 48 of 2 take 29), clusters of 4 and 8 do as long as they cover at most 128 SMs.
FZ_API int fz_gemm_tc_rows_splits(int M, int N, int K) {
  if (M <= BM || N < 256) return 1;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  const long long tiles = (long long)((M + BM - 1) / BM) * ((N + 255) / 256);
  const int kblocks = (K + BK - 1) / BK;
  if (2 * tiles > sms) return 1;
  for (int s = 8; s >= 2; s >>= 1)
    if (tiles * s <= (s == 2 ? sms : 128) && kblocks / 8 >= s) return s;
  return 1;
}

static int device_sms() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  return sms;
}

// Which many-token kernel takes a product: 0 by the rule below, 1 always one SM per tile, 2 a pair of SMs per tile
// wherever the tile is 256 wide (for measurements and tests; the results differ by nothing but the kernel).
static int g_rows_mode = 0;
FZ_API void fz_gemm_tc_rows_mode(int mode) { g_rows_mode = mode; }

// Does a pair of SMs work on each 256 x 256 tile of this product (M > 128 token rows, not cut along K)? Where the pairs
// have at least half a round of tiles, and the token rows fill the pairs' second halves: an even count of 128-row tiles,
// or so many that the one empty half costs less than the pair gains (measured: 10 to 14 % at 1,024 rows and more).
FZ_API int fz_gemm_tc_rows_pairs(int M, int N, int K) {
  if (M <= BM || N < 256 || g_rows_mode == 1) return 0;
  if (g_rows_mode == 2) return 1;
  const int t128 = (M + BM - 1) / BM;
  const long long tiles = (long long)((t128 + 1) / 2) * ((N + PAIR_BN - 1) / PAIR_BN);
  return ((t128 % 2 == 0 || t128 >= 9) && 4 * tiles >= device_sms()) ? 1 : 0;
}

// The number of K pieces when pairs of SMs work on 256 x 256 tiles of a product that is cut along K (1: not this way).
// Only where the one-SM rule cuts K in two and the 128-row tiles come in an even count (no pair's second half empty):
// the clusters are then (2, 1, 2), as many CTAs as before draw a third fewer bytes each (measured: 29.5 -> 27.6 us for
// 256 x 6144 x 4096, 62.6 -> 54.7 us for 512 x 4096 x 14336). Clusters of (2, 1, 4) do not pack the GPCs: 16 of them
// took 41 us for 256 x 4096 x 4096 where 32 clusters of four one-SM pieces take 24.
FZ_API int fz_gemm_tc_rows_pair_splits(int M, int N, int K) {
  if (g_rows_mode == 1 || fz_gemm_tc_rows_splits(M, N, K) != 2) return 1;
  const int t128 = (M + BM - 1) / BM;
  if (t128 % 2) return 1;
  const long long tiles = (long long)(t128 / 2) * ((N + SPLIT_BN - 1) / SPLIT_BN);
  return tiles * 4 <= 128 ? 2 : 1;
}

// x: [M, K] bf16, w: [N, K] bf16, bias: [N] float32 or null, c: [M, N] float32 (out_dtype 0) or bf16 (1).
static int gemm_tc_impl(const void* x, const void* w, const float* bias, void* c, int out_dtype, int M, int N, int K,
                        const Params& fused, int* err, cudaStream_t stream);

FZ_API int fz_gemm_tc(const void* x, const void* w, const float* bias, void* c, int out_dtype, int M, int N, int K,
                      int* err, cudaStream_t stream) {
  return gemm_tc_impl(x, w, bias, c, out_dtype, M, N, K, Params{}, err, stream);
}

// Can the query/key/value product of M token rows with heads of size hd end in the rotation and the cache write?
// (a 128-feature tile must hold whole heads; up to 32 rows, where the separate rotation kernel costs more than its work:
// with more rows the epilogue's per-token lookups outweigh the launch they save)
FZ_API int fz_gemm_tc_qkv_rope_check(int M, int hd) {
  return (M >= 1 && M <= 32 && hd >= 2 && hd % 2 == 0 && 128 % hd == 0) ? FZ_OK : FZ_BAD_SHAPE;
}

// x: [M, K] bf16; w: [(Hq + 2 Hkv) hd, K] bf16, rows [q heads | k heads | v heads]; bias float32 or null. Rotates the q
// and k heads of every token by its position (pairs j, j + hd / 2; angles from cos_t / sin_t [max_len, hd / 2]) and
// writes q to q_out [M, Hq hd] bf16 and, if `write`, k and v to the token's slot of the paged pools (as the separate
// rotation kernel does, with the same roundings). seq_row < 0: a padding row (q zeros, nothing stored).
FZ_API int fz_gemm_tc_qkv_rope(const void* x, const void* w, const float* bias, int M, int K, const float* cos_t,
                               const float* sin_t, const int* pos, const int* seq_row, const int* table, int mb,
                               void* k_pool, void* v_pool, long long page_stride, int page_size, int write, void* q_out,
                               int Hq, int Hkv, int hd, int max_len, int* err, cudaStream_t stream) {
  if (fz_gemm_tc_qkv_rope_check(M, hd) != FZ_OK || Hq <= 0 || Hkv <= 0 || page_size <= 0) return FZ_BAD_SHAPE;
  Params f{};
  f.rope = 1;
  f.cos_t = cos_t; f.sin_t = sin_t; f.pos = pos; f.seq_row = seq_row; f.table = table; f.mb = mb;
  f.k_pool = (__nv_bfloat16*)k_pool; f.v_pool = (__nv_bfloat16*)v_pool; f.page_stride = page_stride;
  f.page_size = page_size; f.write = write; f.Hq = Hq; f.Hkv = Hkv; f.hd = hd; f.max_len = max_len;
  return gemm_tc_impl(x, w, bias, q_out, FZ_BF16, M, (Hq + 2 * Hkv) * hd, K, f, err, stream);
}

// The best (value, index) of a row over its tiles' partial results, in tile order; out[r] = the index (0 if none).
__global__ void argmax_tiles_kernel(const float* __restrict__ val, const int* __restrict__ idx, int tiles, int* __restrict__ out) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  __shared__ float s_v[32];
  __shared__ int s_i[32];
  const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float x = 0.f;
  int ix = 0x7fffffff;
  for (int t = threadIdx.x; t < tiles; t += blockDim.x) {
    const float v = val[(size_t)r * tiles + t];
    const int i = idx[(size_t)r * tiles + t];
    if (am_better(v, i, x, ix)) { x = v; ix = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ox = __shfl_xor_sync(0xffffffffu, x, o);
    const int oi = __shfl_xor_sync(0xffffffffu, ix, o);
    if (am_better(ox, oi, x, ix)) { x = ox; ix = oi; }
  }
  if (lane == 0) { s_v[warp] = x; s_i[warp] = ix; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    x = lane < nw ? s_v[lane] : 0.f;
    ix = lane < nw ? s_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ox = __shfl_xor_sync(0xffffffffu, x, o);
      const int oi = __shfl_xor_sync(0xffffffffu, ix, o);
      if (am_better(ox, oi, x, ix)) { x = ox; ix = oi; }
    }
    if (lane == 0) out[r] = ix == 0x7fffffff ? 0 : ix;
  }
}

// Can `fz_gemm_tc_argmax` take the product? Few token rows, and so many output tiles that K is not split.
FZ_API int fz_gemm_tc_argmax_check(int M, int N, int K) {
  return (M >= 1 && M <= 128 && N >= 1 && K >= 8 && K % 8 == 0 && fz_gemm_tc_splits(N, K) == 1) ? FZ_OK : FZ_BAD_SHAPE;
}

// ids[m] = argmax_n (x[m] . w[n] + bias[n]), numpy's order, without writing the products out. scratch_val / scratch_idx:
// M * ceil(N / 128) elements each.
FZ_API int fz_gemm_tc_argmax(const void* x, const void* w, const float* bias, int M, int N, int K, float* scratch_val,
                             int* scratch_idx, int* ids, int* err, cudaStream_t stream) {
  if (fz_gemm_tc_argmax_check(M, N, K) != FZ_OK) return FZ_BAD_SHAPE;
  Params f{};
  f.argmax = 1;
  f.am_val = scratch_val;
  f.am_idx = scratch_idx;
  int st = gemm_tc_impl(x, w, bias, scratch_val, FZ_F32, M, N, K, f, err, stream);
  if (st != FZ_OK) return st;
  fz_launch(argmax_tiles_kernel, dim3(M), dim3(256), 0, stream, (const float*)scratch_val, (const int*)scratch_idx,
            (N + BM - 1) / BM, ids);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

// Fused gate/up product and SwiGLU: w is [2 I, K] with rows in blocks of 128 = [64 gate rows | 64 up rows] of the same 64
// features (bias packed the same way, or null); out is bf16 [M, I] = silu(x . gate^T) * (x . up^T). I % 64 == 0.
FZ_API int fz_gemm_tc_swiglu(const void* x, const void* w_packed, const float* bias_packed, void* out, int M, int I, int K,
                             int* err, cudaStream_t stream) {
  if (I <= 0 || I % 64) return FZ_BAD_SHAPE;
  if (((uintptr_t)out) & 15) return FZ_BAD_ALIGNMENT;
  Params f{};
  f.swiglu = 1;
  return gemm_tc_impl(x, w_packed, bias_packed, out, FZ_BF16, M, 2 * I, K, f, err, stream);
}

static int gemm_tc_impl(const void* x, const void* w, const float* bias, void* c, int out_dtype, int M, int N, int K,
                        const Params& fused, int* err, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return FZ_OK;
  int st = fz_gemm_tc_check(x, w, M, N, K);
  if (st != FZ_OK) return st;
  if (out_dtype != FZ_F32 && out_dtype != FZ_BF16) return FZ_BAD_DTYPE;
  if (fused.rope && M > 32) return FZ_BAD_SHAPE;
  Params p = fused;
  p.c_f32 = out_dtype == FZ_F32 ? (float*)c : nullptr;
  p.c_bf16 = out_dtype == FZ_BF16 ? (__nv_bfloat16*)c : nullptr;
  p.bias = bias; p.err = err; p.rows = M; p.feats = N; p.K = K;
  p.splits = 1;
  p.vec_ok = (N % 8 == 0 && ((uintptr_t)c & 15) == 0) ? 1 : 0;
  CUtensorMap ma, mb;
  if (M <= 128) {
    // swap mode: W rows are the 128 lanes, the token rows are the instruction's N
    const int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
    p.swap = 1;
    p.stages = pick_stages(bn);
    const int tiles = (N + BM - 1) / BM;
    p.splits = fz_gemm_tc_splits(N, K);
    {
      // A CTA that walks few k-blocks gains nothing from a ring deeper than half of them, and the shared memory it
      // leaves free lets blocks of the kernel after this one become resident (and fetch their weights) earlier:
      // measured on the O product of a decode step (8 k-blocks per CTA, 5 -> 4 stages), two engines alternating in one
      // process: batch 1 3.249 -> 3.212 ms per step, batch 8 3.908 -> 3.898; the same on the down product (28 k-blocks
      // per CTA) or on the q/k/v product lost.
      const int per_cta = ((K + BK - 1) / BK + p.splits - 1) / p.splits, enough = per_cta / 2 < 3 ? 3 : per_cta / 2;
      if (p.stages > enough) p.stages = enough;
    }
    if ((st = get_map_bf16(w, N, K, BM, &ma)) != FZ_OK) return st;
    if ((st = get_map_bf16(x, M, K, bn, &mb)) != FZ_OK) return st;
    dim3 grid(tiles, 1, p.splits);
    switch (bn) {
      case 16: return launch<16>(ma, mb, p, grid, stream);
      case 32: return launch<32>(ma, mb, p, grid, stream);
      case 64: return launch<64>(ma, mb, p, grid, stream);
      default: return launch<128>(ma, mb, p, grid, stream);
    }
  }
  // rows mode: token rows are the 128 lanes; persistent CTAs with two accumulators
  p.swap = 0;
  int bn = N >= 256 ? 256 : N >= 128 ? 128 : 64;     // with the fused SwiGLU N = 2 I >= 128, so a tile holds whole blocks
  if (bn == 256 && !p.swiglu) {
    // So few 128 x 256 tiles that the SMs are not half used, and a K worth cutting: the tiles' K ranges are cut so that
    // about one CTA per SM works (see `gemm_tc_rows_split_kernel`). The count follows from (M, N, K) of the product.
    const int pair_splits = fz_gemm_tc_rows_pair_splits(M, N, K);
    if (pair_splits > 1) {      // the same with a pair of SMs on each 256 x 256 tile
      p.splits = pair_splits;
      p.stages = (200 * 1024) / ((BM + SPLIT_BN / 2) * BK * 2);
      if ((st = get_map_bf16(x, M, K, BM, &ma)) != FZ_OK) return st;
      if ((st = get_map_bf16(w, N, K, SPLIT_BN / 2, &mb)) != FZ_OK) return st;
      return launch_rows_split<true>(ma, mb, p, (M + 2 * BM - 1) / (2 * BM), (N + SPLIT_BN - 1) / SPLIT_BN, stream);
    }
    const int splits = fz_gemm_tc_rows_splits(M, N, K);
    if (splits > 1) {
      p.splits = splits;
      const int stage = (BM + SPLIT_BN) * BK * 2;
      p.stages = (200 * 1024) / stage;
      if ((st = get_map_bf16(x, M, K, BM, &ma)) != FZ_OK) return st;
      if ((st = get_map_bf16(w, N, K, SPLIT_BN, &mb)) != FZ_OK) return st;
      return launch_rows_split<false>(ma, mb, p, (M + BM - 1) / BM, (N + SPLIT_BN - 1) / SPLIT_BN, stream);
    }
  }
  if (bn == 256 && !p.swiglu) {
    // Few token rows: when the 256-wide tiles do not fill the SMs even once, the narrowest width that still fits one
    // round is the fastest (256 x 4096 x 4096 is 32 tiles of 256 columns for 148 SMs, but 52 of 160). Not below 160:
    // a 128-wide instruction reads its operands from shared memory at the rate the tensor core consumes them and runs
    // at about half speed. With more than one round the widest tile stays: measured at 2,048 rows, 160-wide tiles in
    // three rounds (60 -> 72 us) lose against 256-wide ones in two, whatever the count of rounds says.
    static int sms = 0;
    if (sms == 0) {
      int dev = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      if (sms <= 0) sms = 148;
    }
    const long long tm = (M + BM - 1) / BM;
    if (tm * ((N + 255) / 256) < sms) {
      for (int cand : {224, 192, 160})
        if (tm * ((N + cand - 1) / cand) <= sms) bn = cand;
    }
  }
  if (bn == 256 && fz_gemm_tc_rows_pairs(M, N, K)) {
    // many token rows: a pair of SMs on every 256 x 256 tile (see `gemm_tc_rows_pair_kernel`)
    p.stages = (200 * 1024) / ((BM + PAIR_BN / 2) * BK * 2);
    if ((st = get_map_bf16(x, M, K, BM, &ma)) != FZ_OK) return st;
    if ((st = get_map_bf16(w, N, K, PAIR_BN / 2, &mb)) != FZ_OK) return st;
    return launch_rows_pair(ma, mb, p, (M + 2 * BM - 1) / (2 * BM), (N + PAIR_BN - 1) / PAIR_BN, device_sms(), stream);
  }
  {
    const int stage = (BM + bn) * BK * 2;
    const int st_n = (200 * 1024) / stage;
    p.stages = st_n < 2 ? 2 : (st_n > 8 ? 8 : st_n);
  }
  if ((st = get_map_bf16(x, M, K, BM, &ma)) != FZ_OK) return st;
  if ((st = get_map_bf16(w, N, K, bn, &mb)) != FZ_OK) return st;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + bn - 1) / bn;
  switch (bn) {
    case 256: return launch_rows<256>(ma, mb, p, tiles_m, tiles_n, stream);
    case 224: return launch_rows<224>(ma, mb, p, tiles_m, tiles_n, stream);
    case 192: return launch_rows<192>(ma, mb, p, tiles_m, tiles_n, stream);
    case 160: return launch_rows<160>(ma, mb, p, tiles_m, tiles_n, stream);
    case 128: return launch_rows<128>(ma, mb, p, tiles_m, tiles_n, stream);
    default: return launch_rows<64>(ma, mb, p, tiles_m, tiles_n, stream);
  }
}

#ifdef FZ_TIMELINE
FZ_TIMELINE_READER(gemm_tc)
#endif
