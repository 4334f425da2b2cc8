// Paged attention for decoded tokens and short portions, bf16 cache, on tensor cores, split along the keys.
//
// All G = Hq / Hkv query heads of a kv head are the rows of the 16-row MMA tile, so keys and values are read once for the
// whole group (the reference's default decode kernel lays the group out the same way:
// fusezap/device/cuda_kernels/attention.py:860-1043). S = Q K^T and O += P V with mma.sync m16n8k16 on 16 keys at a
// time, softmax online in the exp2 domain with float32 max and sum, P rounded to bf16 for the second product. The key
// axis is cut at fixed positions (the same for every request and batch: a row's sums have one order that depends on
// its own position only); each piece leaves its unnormalised O and (max, sum) in a float32 scratch, and a combine
// kernel merges a row's pieces in rising order and normalises. Rows of portions with at least `long_from` tokens are
// left to the prefill kernel.
//
// Two variants. `attn_decode_units_kernel` (page sizes 8, 16 and multiples of 16; see there): a persistent grid whose
// warps each take an equal share of the step's 64-key units and fetch them with TMA tile loads through rings of their
// own; this is what keeps HBM3e busy at small and large batches alike. `attn_decode_kernel` (any page size): grid
// (partitions of 256 keys, kv heads, token rows); a CTA gathers its partition in 64-key tiles with cp.async through a
// three-stage ring, warp w owns keys 16 w .. 16 w + 15 of each tile, and the four warps' results are merged in warp order.
#include "attn_mma.cuh"
#include "tma.cuh"
#include <math.h>

namespace {
using namespace fzattn;

constexpr int PART = 256;      // keys per partition
constexpr int TILE = 64;       // keys per shared-memory tile
constexpr int THREADS = 128;
constexpr int STAGES = 3;      // key / value tiles in flight

// One warp, 16 keys: S = Q K^T (16 x 16), online softmax update, O += P V. `kaddr(row, chunk)` / `vaddr(row, chunk)`
// give the shared-memory address of the 16-byte chunk `chunk` of key row `row` (0..15) of the group.
template <int HD, typename KAddr, typename VAddr>
__device__ __forceinline__ void attend16(const uint32_t (&qf)[HD / 16][4], KAddr kaddr, VAddr vaddr, int key_first, int lo,
                                         int p, float scale_log2, float (&o)[HD / 8][4], float (&m_run)[2],
                                         float (&l_run)[2], int lane) {
  constexpr int KSTEPS = HD / 16, NB = HD / 8;
  float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
  const int mi = lane >> 3;
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    uint32_t kf[4];
    ldmatrix_x4(kf, kaddr((mi >> 1) * 8 + (lane & 7), ks * 2 + (mi & 1)));
    mma_bf16(s[0], qf[ks], kf[0], kf[1]);
    mma_bf16(s[1], qf[ks], kf[2], kf[3]);
  }
  const int key_base = key_first + 2 * (lane & 3);
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int key = key_base + 8 * j + (e & 1);
      const bool valid = key >= lo && key <= p;
      s[j][e] = valid ? s[j][e] * scale_log2 : -INFINITY;
      mx[e >> 1] = fmaxf(mx[e >> 1], s[j][e]);
    }
  uint32_t pf[4];
  float corr[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    const float mn = fmaxf(m_run[h], mx[h]);
    const float mu = mn == -INFINITY ? 0.f : mn;      // no visible key yet: every exponent below is exp2(-inf) = 0
    corr[h] = exp2f(m_run[h] - mu);
    m_run[h] = mn;
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const float e0 = exp2f(s[j][2 * h] - mu), e1 = exp2f(s[j][2 * h + 1] - mu);
      sum += e0 + e1;
      pf[2 * j + h] = pack_bf16(e0, e1);
    }
    l_run[h] = l_run[h] * corr[h] + sum;
  }
#pragma unroll
  for (int i = 0; i < NB; ++i) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
#pragma unroll
  for (int nb = 0; nb < NB; nb += 2) {
    uint32_t vf[4];
    ldmatrix_x4_trans(vf, vaddr((mi & 1) * 8 + (lane & 7), nb + (mi >> 1)));
    mma_bf16(o[nb], pf, vf[0], vf[1]);
    mma_bf16(o[nb + 1], pf, vf[2], vf[3]);
  }
}

// The same for groups of at most 8 query heads, with the products transposed so that no MMA row is padding: the 16 keys
// are the rows of S^T = K Q^T (16 x 8 heads), and O^T += V^T P^T has 16 head dimensions as rows and the heads as its 8
// columns. Half the MMAs, half the accumulators and half the exponentials of `attend16`. A thread holds, of S^T, keys
// lane / 4 and lane / 4 + 8 for heads 2 (lane % 4) + {0, 1}; of O^T block i, dimensions 16 i + lane / 4 (+ 8) for the
// same two heads. m_run / l_run are per head (l_run: this thread's keys only; the caller adds the lanes of a head up).
// qf[ks] = Q[head lane / 4][16 ks + 2 (lane % 4) + {0, 1}] and the same + 8 (zero for heads past the group).
template <int HD, typename KAddr, typename VAddr>
__device__ __forceinline__ void attend16_small(const uint32_t (&qf)[HD / 16][2], KAddr kaddr, VAddr vaddr, int key_first,
                                               int lo, int p, float scale_log2, float (&o)[HD / 16][4], float (&m_run)[2],
                                               float (&l_run)[2], int lane) {
  constexpr int KSTEPS = HD / 16, DB = HD / 16;
  float s[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f};    // even and odd k-steps: two chains in flight
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ks += 2) {
    uint32_t kf[4], kg[4];
    ldmatrix_x4(kf, kaddr(lane & 15, ks * 2 + (lane >> 4)));
    ldmatrix_x4(kg, kaddr(lane & 15, ks * 2 + 2 + (lane >> 4)));
    mma_bf16(s, kf, qf[ks][0], qf[ks][1]);
    mma_bf16(s2, kg, qf[ks + 1][0], qf[ks + 1][1]);
  }
  const int key_a = key_first + (lane >> 2), key_b = key_a + 8;
  const bool va = key_a >= lo && key_a <= p, vb = key_b >= lo && key_b <= p;
  s[0] = va ? (s[0] + s2[0]) * scale_log2 : -INFINITY;
  s[1] = va ? (s[1] + s2[1]) * scale_log2 : -INFINITY;
  s[2] = vb ? (s[2] + s2[2]) * scale_log2 : -INFINITY;
  s[3] = vb ? (s[3] + s2[3]) * scale_log2 : -INFINITY;
  float corr[2], mu[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    float mx = fmaxf(s[j], s[j + 2]);
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
    const float mn = fmaxf(m_run[j], mx);
    mu[j] = mn == -INFINITY ? 0.f : mn;        // no visible key yet: every exponent below is exp2(-inf) = 0
    corr[j] = exp2f(m_run[j] - mu[j]);
    m_run[j] = mn;
  }
  const float e0 = exp2f(s[0] - mu[0]), e1 = exp2f(s[1] - mu[1]), e2 = exp2f(s[2] - mu[0]), e3 = exp2f(s[3] - mu[1]);
  l_run[0] = l_run[0] * corr[0] + (e0 + e2);
  l_run[1] = l_run[1] * corr[1] + (e1 + e3);
  // P (keys x heads, in the accumulator layout) -> P^T as the B operand: one 8 x 8 transpose per 8 keys
  uint32_t pb0, pb1;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(pb0) : "r"(pack_bf16(e0, e1)));
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(pb1) : "r"(pack_bf16(e2, e3)));
#pragma unroll
  for (int i = 0; i < DB; ++i) { o[i][0] *= corr[0]; o[i][1] *= corr[1]; o[i][2] *= corr[0]; o[i][3] *= corr[1]; }
#pragma unroll
  for (int i = 0; i < DB; ++i) {
    uint32_t vf[4];      // V^T: dimensions 16 i .. + 15 as rows, the 16 keys as columns
    ldmatrix_x4_trans(vf, vaddr((lane & 7) + 8 * (lane >> 4), 2 * i + ((lane >> 3) & 1)));
    mma_bf16(o[i], vf, pb0, pb1);
  }
}

// Merges the four warps' (max, sum, O) in warp order and writes the partition's unnormalised O and (max, sum).
// `scratch` is shared memory for [4][16][HD] + [4][16][2] floats; the caller has synchronised the block before.
template <int HD>
__device__ __forceinline__ void merge_and_store(float* scratch, const float (&o)[HD / 8][4], float (&m_run)[2], float (&l_run)[2],
                                                float* __restrict__ part_o, float* __restrict__ ml_out, int n, int Hq,
                                                int kvh, int G, int NP, int part, int tid) {
  constexpr int NB = HD / 8, THREADS = 128;
  const int warp = tid >> 5, lane = tid & 31;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  float* m_o = scratch;                             // [4 warps][16 rows][HD + 4]: the pad spreads the rows over the banks
  constexpr int LD = HD + 4;
  float* m_ml = m_o + 4 * 16 * LD;                  // [4][16][2]
  const int r0 = lane >> 2;
#pragma unroll
  for (int i = 0; i < NB; ++i) {
    const int d = 8 * i + 2 * (lane & 3);
    float* w0 = m_o + ((size_t)warp * 16 + r0) * LD + d;
    w0[0] = o[i][0]; w0[1] = o[i][1];
    w0[8 * LD] = o[i][2]; w0[8 * LD + 1] = o[i][3];
  }
  if ((lane & 3) == 0) {
    m_ml[(warp * 16 + r0) * 2] = m_run[0]; m_ml[(warp * 16 + r0) * 2 + 1] = l_run[0];
    m_ml[(warp * 16 + r0 + 8) * 2] = m_run[1]; m_ml[(warp * 16 + r0 + 8) * 2 + 1] = l_run[1];
  }
  __syncthreads();
  for (int e = tid; e < G * HD; e += THREADS) {
    const int g = e / HD, d = e - g * HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, m_ml[(w * 16 + g) * 2]);
    const float Mu = M == -INFINITY ? 0.f : M;
    float acc = 0.f, L = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = exp2f(m_ml[(w * 16 + g) * 2] - Mu);
      acc += m_o[((size_t)w * 16 + g) * LD + d] * f;
      L += m_ml[(w * 16 + g) * 2 + 1] * f;
    }
    part_o[(((size_t)n * Hq + (size_t)kvh * G + g) * NP + part) * HD + d] = acc;
    if (d == 0) { ml_out[(size_t)g * NP * 2] = M; ml_out[(size_t)g * NP * 2 + 1] = L; }
  }
}

template <int HD>
__global__ void __launch_bounds__(THREADS)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                   const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ pos,
                   const int* __restrict__ seq_row, const int* __restrict__ seg, const int* __restrict__ table, int mb,
                   long long page_stride, int page_size, float* __restrict__ part_o, float* __restrict__ part_ml,
                   int Hq, int Hkv, float scale_log2, int window, int long_from) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  constexpr int KSTEPS = HD / 16;      // k-steps of Q K^T
  constexpr int NB = HD / 8;           // 8-wide output blocks of P V
  extern __shared__ __align__(128) uint8_t smem[];
  // [STAGES][K tile | V tile] then the Q tile; the merge buffers reuse the stages
  constexpr int TILE_BYTES = TILE * HD * 2;
  const uint32_t s_base = smem_u32(smem);
  const uint32_t s_q = s_base + 2 * STAGES * TILE_BYTES;

  const int part = blockIdx.x, kvh = blockIdx.y, n = blockIdx.z, NP = gridDim.x;
  const int G = Hq / Hkv;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row = seq_row[n];
  if (row < 0) return;
  if (seg[row * 4 + 1] >= long_from) return;      // a long portion: the prefill kernel's rows
  const int p = pos[n];
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int k_begin = max(part * PART, lo & ~(TILE - 1)), k_end = min((part + 1) * PART, p + 1);   // [k_begin, k_end)
  float* ml_out = part_ml + (((size_t)n * Hq + (size_t)kvh * G) * NP + part) * 2;
  if (k_begin >= k_end) {   // nothing of this row in this partition
    for (int g = tid; g < G; g += THREADS) { ml_out[(size_t)g * NP * 2] = -INFINITY; ml_out[(size_t)g * NP * 2 + 1] = 0.f; }
    return;
  }
  const int* trow = table + (size_t)row * mb;
  const long long head_off = (long long)kvh * page_size * HD;

  // Q: G rows of HD, zero rows up to 16, swizzled
  {
    const __nv_bfloat16* qrow = q + (size_t)n * Hq * HD + (size_t)kvh * G * HD;
    for (int e = tid; e < 16 * (HD / 8); e += THREADS) {
      const int r = e / (HD / 8), c = e - r * (HD / 8);
      cp_async16(s_q + swz<HD>(r, c), qrow + (size_t)r * HD + c * 8, r < G);
    }
  }
  const int ntiles = (k_end - k_begin + TILE - 1) / TILE;
  auto issue = [&](int t) {      // one commit group per call, empty past the last tile
    if (t < ntiles) {
      const uint32_t st = s_base + (t % STAGES) * 2 * TILE_BYTES;
      load_kv_tile<HD, TILE, THREADS>(st, st + TILE_BYTES, k_pool, v_pool, trow, page_stride, head_off, page_size,
                                      k_begin + t * TILE, lo, p, tid);
    }
    cp_async_commit();
  };
#pragma unroll
  for (int t = 0; t < STAGES - 1; ++t) issue(t);

  uint32_t qf[KSTEPS][4];
  float o[NB][4];
#pragma unroll
  for (int i = 0; i < NB; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // rows lane/4 and lane/4 + 8

  for (int t = 0; t < ntiles; ++t) {
    issue(t + STAGES - 1);
    cp_async_wait<STAGES - 1>();      // all but the newest STAGES - 1 groups have landed: tile t is in
    __syncthreads();
    if (t == 0) {
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks)
        ldmatrix_x4(qf[ks], s_q + swz<HD>(lane & 15, ks * 2 + (lane >> 4)));
    }
    const uint32_t sk = s_base + (t % STAGES) * 2 * TILE_BYTES, sv = sk + TILE_BYTES;
    attend16<HD>(qf, [&](int r, int c) { return sk + swz<HD>(warp * 16 + r, c); },
                 [&](int r, int c) { return sv + swz<HD>(warp * 16 + r, c); }, k_begin + t * TILE + warp * 16, lo, p,
                 scale_log2, o, m_run, l_run, lane);
    __syncthreads();   // the stage may be refilled
  }
  merge_and_store<HD>((float*)smem, o, m_run, l_run, part_o, ml_out, n, Hq, kvh, G, NP, part, tid);
}

// ---------------------------------------------------------------------------------------------- TMA variant
// Key positions are cut into *units*, the same for every request and every batch: keys [0, 4096) in units of 64, later
// keys in units of 256. One warp computes one unit on its own (its 16-key groups one after the other, online softmax)
// and writes the unit's unnormalised O and (max, sum) from its registers; nothing is merged inside the kernel, so a
// row's arithmetic depends on its own position only. The grid is persistent: all units of all (row, kv head) pairs
// of the step are numbered (row, then kv head, then position), and warp w of W takes the units [T w / W, T (w + 1) / W),
// so the SMs stay equally loaded whatever the batch and the contexts are. Every warp runs a TMA ring of its own
// (NSTAGE groups of 16 keys, K and V) that runs ahead across unit boundaries: the loads of the next unit are in flight
// while this one's partial is written.
//
// kv_map: the cache slot's pool seen as a row-major [pages * 2 * Hkv * page_size, HD] bf16 array (row of key `off` of kv
// head `kvh` of page `pg`: pg * 2 Hkv bs + kvh * bs + off; its value row: + Hkv * bs), boxes of BOX rows x 64 columns.
// Shared memory per warp: NSTAGE x [K | V], each HD / 64 column halves of [16 rows][128 bytes], swizzled by TMA.
constexpr int UNIT_SMALL = 64, UNIT_BIG = 256, SMALL_UNITS = 64;
constexpr int SMALL_KEYS = UNIT_SMALL * SMALL_UNITS;
constexpr int MAX_UNIT_ROWS = 4096;      // token rows the unit kernel numbers in shared memory

__host__ __device__ __forceinline__ int unit_of(int key) {
  return key < SMALL_KEYS ? key / UNIT_SMALL : SMALL_UNITS + (key - SMALL_KEYS) / UNIT_BIG;
}
__host__ __device__ __forceinline__ int unit_start(int u) {
  return u < SMALL_UNITS ? u * UNIT_SMALL : SMALL_KEYS + (u - SMALL_UNITS) * UNIT_BIG;
}
__host__ __device__ __forceinline__ int unit_len(int u) { return u < SMALL_UNITS ? UNIT_SMALL : UNIT_BIG; }

// Merging the partial result (m2, l2, o2) of a unit into the running (m, l, o) of its block. The unit kernel and the
// combine kernel both merge with exactly these operations, so the bits do not depend on which of them did it.
__device__ __forceinline__ void merge_unit_scalars(float& m, float& l, float m2, float l2, float& fa, float& fb) {
  const float mn = fmaxf(m, m2);
  fa = exp2f(m - mn);
  fb = exp2f(m2 - mn);
  l = __fmaf_rn(l2, fb, __fmul_rn(l, fa));
  m = mn;
}
__device__ __forceinline__ float merge_unit_value(float o, float o2, float fa, float fb) {
  return __fmaf_rn(o2, fb, __fmul_rn(o, fa));
}

// Where a warp stands in its list of units: the unit's row, kv head and key range, and the next 16-key group.
struct UnitCursor {
  int u;            // number of the unit among the step's units
  int n, kvh;       // token row, kv head
  int unit;         // which unit of the key axis
  int p, lo;        // the row attends keys lo .. p
  int key0;         // first key of the unit
  int g, g_end;     // next group of 16 keys in the unit, one past the last
  int page0;        // first block-table entry the unit's groups need ...
  int pages;        // ... and entry page0 + lane of the table (-1 past the row's position), one per lane
  int first_new;    // the first position of the row's request that this step writes: keys below it are from earlier steps
  bool valid;
};

template <int HD, int BOX, int NSTAGE, int MINB, bool SMALLG>
__global__ void __launch_bounds__(THREADS, MINB)
attn_decode_units_kernel(const __grid_constant__ CUtensorMap kv_map, const __nv_bfloat16* __restrict__ q,
                         const int* __restrict__ pos, const int* __restrict__ seq_row, const int* __restrict__ seg,
                         const int* __restrict__ table, int mb, int page_size, float* __restrict__ part_o,
                         float* __restrict__ part_ml, int N, int Hq, int Hkv, int NPU, float scale_log2, int window,
                         int long_from, int single, int* err) {
  // SMALLG (at most 8 query heads per kv head): the transposed products of `attend16_small`
  constexpr int KSTEPS = HD / 16, OB = SMALLG ? HD / 16 : HD / 8, QW = SMALLG ? 2 : 4, HALVES = HD / 64;
  constexpr int HALF_BYTES = 16 * 128;                 // one column half of a 16-key group
  constexpr int KV_BYTES = HALVES * HALF_BYTES;        // keys (or values) of a group
  constexpr int STAGE_BYTES = 2 * KV_BYTES;
  constexpr int WARP_BYTES = NSTAGE * STAGE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t s_base = smem_u32(smem);
  uint64_t* bars = (uint64_t*)(smem + 4 * WARP_BYTES);                   // [4 warps][NSTAGE]
  int* s_pre = (int*)(bars + 4 * NSTAGE);                                // [N + 1]: units before row n

  // Prologue that depends on nothing another kernel writes: the barriers.
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int i = 0; i < 4 * NSTAGE; ++i) fztma::mbar_init(&bars[i], 1);
    fztma::mbar_init_fence();
  }
  __syncthreads();
  fz_grid_launch_dependents();
  // What follows up to the wait reads only the step's metadata (positions, rows, block tables): the host wrote it before
  // the step's first kernel started and no kernel changes it, so it may be read while the kernel before this one runs.

  const int G = Hq / Hkv;
  // units of every row (0 for padding rows and for rows of long portions), then their running sum
  for (int n = tid; n < N; n += THREADS) {
    // `single`: every portion of the step is one token, so no row belongs to a long portion and the portion's record
    // need not be asked for (a load that could only start when the row number has arrived)
    const int row = seq_row[n];
    const int p = pos[n];
    int cnt = 0;
    if (row >= 0 && (single || seg[row * 4 + 1] < long_from)) {
      const int lo = window > 0 ? max(0, p - window + 1) : 0;
      cnt = (unit_of(p) - unit_of(lo) + 1) * Hkv;
    }
    s_pre[n + 1] = cnt;
  }
  if (tid == 0) s_pre[0] = 0;
  __syncthreads();
  if (warp == 0) {
    int carry = 0;
    for (int base = 0; base < N; base += 32) {
      const int i = base + lane;
      int v = i < N ? s_pre[i + 1] : 0;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += t;
      }
      if (i < N) s_pre[i + 1] = v + carry;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
  }
  __syncthreads();
  // from here on the warps go their own ways: no block-wide barrier below
  const long long T = s_pre[N];
  const long long gw = (long long)blockIdx.x * 4 + warp, W = (long long)gridDim.x * 4;
  const int u_begin = (int)(T * gw / W), u_end = (int)(T * (gw + 1) / W);
  if (u_begin >= u_end) { fz_grid_wait(); return; }

  auto load_unit = [&](UnitCursor& c, int u, int n_hint, bool with_pages) {
    c.u = u;
    c.valid = u < u_end;
    if (!c.valid) return;
    int n = n_hint;
    if (!(s_pre[n] <= u && u < s_pre[n + 1])) {      // the largest n with s_pre[n] <= u
      int a = 0, b = N - 1;
      while (a < b) {
        const int mid = (a + b + 1) >> 1;
        if (s_pre[mid] <= u) a = mid; else b = mid - 1;
      }
      n = a;
    }
    const int r = u - s_pre[n], per_head = (s_pre[n + 1] - s_pre[n]) / Hkv;
    c.n = n;
    c.kvh = r / per_head;
    c.p = pos[n];
    c.lo = window > 0 ? max(0, c.p - window + 1) : 0;
    c.unit = unit_of(c.lo) + (r - c.kvh * per_head);
    c.key0 = unit_start(c.unit);
    c.g = c.lo > c.key0 ? (c.lo - c.key0) >> 4 : 0;
    c.g_end = min(unit_len(c.unit) >> 4, ((c.p - c.key0) >> 4) + 1);
    // the unit's block-table entries, one per lane (at most 32: 256 keys in pages of 8), asked for now and used
    // when the unit's loads are issued
    if (!with_pages) return;
    const int row = seq_row[n];
    c.first_new = single ? c.p : seg[row * 4 + 2];      // a single token is its portion's first
    c.page0 = (c.key0 + 16 * c.g) / page_size;
    const int pi = c.page0 + lane;
    c.pages = (pi < mb && pi * page_size <= c.p) ? __ldg(table + (size_t)row * mb + pi) : -1;
  };

  const uint32_t s_warp = s_base + warp * WARP_BYTES;
  uint64_t* wbars = bars + warp * NSTAGE;
  const int rows_per_page = 2 * Hkv * page_size;
  // keys and values are read once per step: they should leave L2 before the partial results, which are read again
  const uint64_t stream_once = fztma::l2_evict_first();
  auto issue = [&](const UnitCursor& c, int stage) {        // the whole warp (the pages sit in the lanes); lane 0 loads
    const int key0 = c.key0 + 16 * c.g;
    uint64_t* bar = &wbars[stage];
    int rows[16 / BOX];
    uint32_t bytes = 0;
    bool zeroed = false;
#pragma unroll
    for (int sub = 0; sub < 16 / BOX; ++sub) {
      const int key = key0 + sub * BOX;
      rows[sub] = -1;
      const int pi = key / page_size;
      const int page = __shfl_sync(0xffffffffu, c.pages, (pi - c.page0) & 31);
      const bool unseen = key > c.p || key + BOX - 1 < c.lo;     // nothing visible in this box
      if (unseen || page < 0) {
        if (!unseen && lane == 0) atomicOr(err, FZ_ERR_NO_PAGE);
        // The box is not fetched: its part of the stage must hold finite bits (P = 0 times NaN is NaN), so the warp
        // writes zeros there. (Zeroing all stages when the block starts took 0.6 us of every block's start, which
        // counts for the blocks that become resident only when the kernel before this one leaves their SM.)
        uint8_t* st = smem + (size_t)warp * WARP_BYTES + (size_t)stage * STAGE_BYTES;
#pragma unroll
        for (int h = 0; h < 2 * HALVES; ++h)            // the K halves, then the V halves
          for (int e = lane; e < BOX * 128 / 16; e += 32) ((uint4*)(st + h * HALF_BYTES + sub * BOX * 128))[e] = make_uint4(0u, 0u, 0u, 0u);
        zeroed = true;
        continue;
      }
      rows[sub] = page * rows_per_page + c.kvh * page_size + (key - pi * page_size);
      bytes += 2 * HALVES * BOX * 128;
    }
    if (zeroed) {       // (warp-uniform) ordinary stores before later bulk copies into the same bytes
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
    }
    if (lane != 0) return;
    fztma::mbar_expect_tx(bar, bytes);
    const uint32_t sk = s_warp + stage * STAGE_BYTES, sv = sk + KV_BYTES, b = smem_u32(bar);
#pragma unroll
    for (int sub = 0; sub < 16 / BOX; ++sub) {
      if (rows[sub] < 0) continue;
#pragma unroll
      for (int h = 0; h < HALVES; ++h) {
        fztma::tma_load_2d_u32_hint(sk + h * HALF_BYTES + sub * BOX * 128, &kv_map, b, 64 * h, rows[sub], stream_once);
        fztma::tma_load_2d_u32_hint(sv + h * HALF_BYTES + sub * BOX * 128, &kv_map, b, 64 * h, rows[sub] + Hkv * page_size, stream_once);
      }
    }
  };

  // where the arithmetic stands, where the loads stand, and the unit after that one (its block-table entries are on
  // their way while the loads of the unit before it are issued)
  UnitCursor cc, ci, cn;
  load_unit(ci, u_begin, 0, true);
  cc = ci;             // (the arithmetic never looks at the pages)
  load_unit(cn, u_begin + 1, ci.n, true);
  auto advance_loads = [&]() {
    if (++ci.g >= ci.g_end) {
      ci = cn;
      if (ci.valid) load_unit(cn, ci.u + 1, ci.n, true);
    }
  };
  int issued = 0, consumed = 0;
  // Keys and values below the first position that this step writes for the row's request were written by earlier steps
  // (a step starts only after the one before it has finished, and nothing in a step writes below that position): the
  // loads of such groups go out before the wait, so the first stages fill while the kernel before this one finishes.
  while (ci.valid && issued < NSTAGE && ci.key0 + 16 * ci.g + 15 < ci.first_new) {
    issue(ci, issued);
    ++issued;
    advance_loads();
  }
  fz_grid_wait();      // the queries and the newest keys and values come from the kernels before
  int q_n = -1, q_kvh = -1;
  uint32_t qf[KSTEPS][QW];
  float o[OB][4];
  float m_run[2], l_run[2];
  float blk_o[OB][4], blk_m[2], blk_l[2];       // the block that is being merged from this warp's own units
  bool fresh = true;
  while (cc.valid) {
    while (ci.valid && issued - consumed < NSTAGE) {
      issue(ci, issued % NSTAGE);
      ++issued;
      advance_loads();
    }
    if (cc.n != q_n || cc.kvh != q_kvh) {
      // another row or kv head: its G query heads, read from global memory straight into the MMA fragments
      q_n = cc.n; q_kvh = cc.kvh;
      const uint32_t* qw = (const uint32_t*)(q + ((size_t)q_n * Hq + (size_t)q_kvh * G) * HD);
      const int r0 = lane >> 2, cw = lane & 3;
      if constexpr (SMALLG) {
        // B operand (Q^T): head lane / 4, dimensions 2 (lane % 4) + {0, 1} and + 8 of every 16; zero past the group
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
          qf[ks][0] = r0 < G ? qw[(r0 * HD + 16 * ks) / 2 + cw] : 0u;
          qf[ks][1] = r0 < G ? qw[(r0 * HD + 16 * ks + 8) / 2 + cw] : 0u;
        }
      } else {
        // A operand: lane l holds rows (heads) l / 4 and l / 4 + 8, columns 2 (l % 4) + {0, 1} and + 8 of every 16
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
          qf[ks][0] = r0 < G ? qw[(r0 * HD + 16 * ks) / 2 + cw] : 0u;
          qf[ks][1] = r0 + 8 < G ? qw[((r0 + 8) * HD + 16 * ks) / 2 + cw] : 0u;
          qf[ks][2] = r0 < G ? qw[(r0 * HD + 16 * ks + 8) / 2 + cw] : 0u;
          qf[ks][3] = r0 + 8 < G ? qw[((r0 + 8) * HD + 16 * ks + 8) / 2 + cw] : 0u;
        }
      }
    }
    if (fresh) {
#pragma unroll
      for (int i = 0; i < OB; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
      m_run[0] = m_run[1] = -INFINITY;
      l_run[0] = l_run[1] = 0.f;
      fresh = false;
    }
    const int stage = consumed % NSTAGE;
    if (!__all_sync(0xffffffffu, fztma::mbar_wait(&wbars[stage], (consumed / NSTAGE) & 1))) {
      if (lane == 0) atomicOr(err, FZ_ERR_WAIT_TIMEOUT);
      return;
    }
    const uint32_t sk = s_warp + stage * STAGE_BYTES, sv = sk + KV_BYTES;
    // chunk c of row r: column half c >> 3, 16-byte chunk (c & 7) ^ (r & 7) of the 128-byte row (TMA's swizzle)
    auto kaddr = [&](int r, int c) { return sk + (c >> 3) * HALF_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4); };
    auto vaddr = [&](int r, int c) { return sv + (c >> 3) * HALF_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4); };
    if constexpr (SMALLG) attend16_small<HD>(qf, kaddr, vaddr, cc.key0 + 16 * cc.g, cc.lo, cc.p, scale_log2, o, m_run, l_run, lane);
    else attend16<HD>(qf, kaddr, vaddr, cc.key0 + 16 * cc.g, cc.lo, cc.p, scale_log2, o, m_run, l_run, lane);
    __syncwarp();        // every lane has read the stage: it may be refilled
    ++consumed;
    if (cc.g + 1 >= cc.g_end) {
      // The unit is complete. Its sum of weights over all lanes that hold keys of a head:
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        if constexpr (SMALLG) {
          l_run[j] += __shfl_xor_sync(0xffffffffu, l_run[j], 4);
          l_run[j] += __shfl_xor_sync(0xffffffffu, l_run[j], 8);
          l_run[j] += __shfl_xor_sync(0xffffffffu, l_run[j], 16);
        } else {
          l_run[j] += __shfl_xor_sync(0xffffffffu, l_run[j], 1);
          l_run[j] += __shfl_xor_sync(0xffffffffu, l_run[j], 2);
        }
      }
      // The 64-key units of one 256-key block that this warp computes all by itself are merged here, in rising order
      // and with the arithmetic of `merge_unit` (the combine kernel merges a block's units the same way when they
      // come from different warps, so the result does not depend on who computed what); the block then leaves one
      // partial result, marked by a negative sum, in the slot of its first unit.
      int write_unit = cc.unit;
      bool write = true;
      if (cc.unit < SMALL_UNITS) {
        const int bu0 = max(unit_of(cc.lo), cc.unit & ~3), bu1 = min(unit_of(cc.p), cc.unit | 3);
        if (bu1 > bu0 && cc.u - (cc.unit - bu0) >= u_begin && cc.u + (bu1 - cc.unit) < u_end) {
          if (cc.unit == bu0) {
#pragma unroll
            for (int i = 0; i < OB; ++i) { blk_o[i][0] = o[i][0]; blk_o[i][1] = o[i][1]; blk_o[i][2] = o[i][2]; blk_o[i][3] = o[i][3]; }
            blk_m[0] = m_run[0]; blk_m[1] = m_run[1]; blk_l[0] = l_run[0]; blk_l[1] = l_run[1];
          } else {
            float fa[2], fb[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) merge_unit_scalars(blk_m[j], blk_l[j], m_run[j], l_run[j], fa[j], fb[j]);
#pragma unroll
            for (int i = 0; i < OB; ++i)
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int j = SMALLG ? (e & 1) : (e >> 1);
                blk_o[i][e] = merge_unit_value(blk_o[i][e], o[i][e], fa[j], fb[j]);
              }
          }
          write = cc.unit == bu1;
          if (write) {
            write_unit = bu0;
#pragma unroll
            for (int i = 0; i < OB; ++i) { o[i][0] = blk_o[i][0]; o[i][1] = blk_o[i][1]; o[i][2] = blk_o[i][2]; o[i][3] = blk_o[i][3]; }
            m_run[0] = blk_m[0]; m_run[1] = blk_m[1]; l_run[0] = -blk_l[0]; l_run[1] = -blk_l[1];
          }
        }
      }
      if (write) {
        // unnormalised O and (max, sum), straight from the MMA fragments
        const size_t head0 = (size_t)cc.n * Hq + (size_t)cc.kvh * G;
        if constexpr (SMALLG) {
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int g = 2 * (lane & 3) + j;
            if (g < G) {
              const size_t slot = (head0 + g) * NPU + write_unit;
              float* dst = part_o + slot * HD + (lane >> 2);
#pragma unroll
              for (int i = 0; i < OB; ++i) { dst[16 * i] = o[i][j]; dst[16 * i + 8] = o[i][2 + j]; }
              if ((lane >> 2) == 0) *(float2*)(part_ml + slot * 2) = make_float2(m_run[j], l_run[j]);
            }
          }
        } else {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int g = (lane >> 2) + 8 * h;
            if (g < G) {
              const size_t slot = (head0 + g) * NPU + write_unit;
              float* dst = part_o + slot * HD + 2 * (lane & 3);
#pragma unroll
              for (int i = 0; i < OB; ++i) *(float2*)(dst + 8 * i) = make_float2(o[i][2 * h], o[i][2 * h + 1]);
              if ((lane & 3) == 0) *(float2*)(part_ml + slot * 2) = make_float2(m_run[h], l_run[h]);
            }
          }
        }
      }
      fresh = true;
    }
    if (++cc.g >= cc.g_end) load_unit(cc, cc.u + 1, cc.n, false);
  }
}

// One block of 128 or 256 threads per (token row, query head). A thread owns four neighbouring output dimensions (one float4 per
// partial result); the HD / 4 threads that cover a row form a group, and the groups share the row's blocks
// of the key axis out among themselves (a block: the up to four 64-key units of 256 keys below key 4096, either already
// merged by the unit kernel or merged here in rising order with the same arithmetic; a 256-key unit above). The groups'
// results are merged in group order, normalised and rounded to bf16. All (max, sum) pairs of the row are brought into
// shared memory first, so that what a thread loads next never waits on a load before it. Which units a row has follows
// from its position and the window alone, as in the kernel above.
__global__ void __launch_bounds__(256)
attn_combine_units_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                          const int* __restrict__ pos, const int* __restrict__ seq_row, const int* __restrict__ seg,
                          __nv_bfloat16* __restrict__ out, int Hq, int HD, int NPU, int window, int long_from) {
  extern __shared__ float2 s_ml[];             // [units of the row], then the groups' results
  fz_grid_launch_dependents();
  const int n = blockIdx.y, h = blockIdx.x, tid = threadIdx.x;
  const int CT = blockDim.x;
  const int per_row = HD >> 2, groups = CT / per_row;           // threads per row, groups per block
  const int grp = tid / per_row, d4 = (tid - grp * per_row) * 4;
  const int row = seq_row[n];
  const bool skip = row >= 0 && seg[row * 4 + 1] >= long_from;
  const int p = pos[n];
  fz_grid_wait();
  __nv_bfloat16* orow = out + ((size_t)n * Hq + h) * HD;
  if (row < 0) {
    if (grp == 0) *(uint2*)(orow + d4) = make_uint2(0u, 0u);
    return;
  }
  if (skip) return;
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int u0 = unit_of(lo), u1 = unit_of(p), cnt = u1 - u0 + 1;
  const float2* ml = (const float2*)part_ml + ((size_t)n * Hq + h) * NPU + u0;
  const float* po = part_o + (((size_t)n * Hq + h) * NPU + u0) * HD + d4;
  for (int i = tid; i < cnt; i += CT) s_ml[i] = ml[i];
  __syncthreads();
  // The row's blocks are merged in VG chains (chain v: blocks v, v + VG, ...), and the chains then in rising order: VG
  // is the group count of a block of 256 threads, and a block of 128 threads walks two chains per group, so the order
  // of the merges, and with it every bit of the result, does not depend on the block's size.
  const int VG = 256 / per_row, lane_in = tid - grp * per_row;
  float4* s_o = (float4*)(s_ml + cnt + (cnt & 1));              // [VG][per_row]
  float2* s_g = (float2*)(s_o + VG * per_row);                  // [VG]: (max, sum)
  const int n_small = u0 < SMALL_UNITS ? (min(u1, SMALL_UNITS - 1) >> 2) - (u0 >> 2) + 1 : 0;
  const int big0 = max(u0, SMALL_UNITS);
  const int n_items = n_small + (u1 >= SMALL_UNITS ? u1 - big0 + 1 : 0);
  auto merge4 = [](float4& o, const float4& o2, float fa, float fb) {
    o.x = merge_unit_value(o.x, o2.x, fa, fb); o.y = merge_unit_value(o.y, o2.y, fa, fb);
    o.z = merge_unit_value(o.z, o2.z, fa, fb); o.w = merge_unit_value(o.w, o2.w, fa, fb);
  };
  for (int v = grp; v < VG; v += groups) {
    float M = -INFINITY, L = 0.f;
    float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = v; k < n_items; k += VG) {
      float Mb, Lb;
      float4 Ob;
      if (k < n_small) {
        const int b = (u0 >> 2) + k;
        const int i0 = max(u0, 4 * b) - u0, i1 = min(u1, 4 * b + 3) - u0;       // the block's units, relative to u0
        const float2 first = s_ml[i0];
        Mb = first.x; Lb = fabsf(first.y);
        if (first.y < 0.f || i1 == i0) {
          Ob = *(const float4*)(po + (size_t)i0 * HD);
        } else {                        // not merged by the unit kernel: the block's units one by one, loads first
          float4 v[4];
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (i0 + j <= i1) v[j] = *(const float4*)(po + (size_t)(i0 + j) * HD);
          Ob = v[0];
#pragma unroll
          for (int j = 1; j < 4; ++j) {
            if (i0 + j <= i1) {
              const float2 next = s_ml[i0 + j];
              float fa, fb;
              merge_unit_scalars(Mb, Lb, next.x, next.y, fa, fb);
              merge4(Ob, v[j], fa, fb);
            }
          }
        }
      } else {
        const int i = big0 + (k - n_small) - u0;
        const float2 v = s_ml[i];
        Mb = v.x; Lb = v.y;
        Ob = *(const float4*)(po + (size_t)i * HD);
      }
      float fa, fb;
      merge_unit_scalars(M, L, Mb, Lb, fa, fb);
      merge4(O, Ob, fa, fb);
    }
    s_o[v * per_row + lane_in] = O;
    if (lane_in == 0) s_g[v] = make_float2(M, L);
  }
  __syncthreads();
  if (grp != 0) return;
  float M = s_g[0].x, L = s_g[0].y;            // (chain 0 holds the row's first block: never empty)
  float4 O = s_o[tid];
  for (int k = 1; k < VG; ++k) {
    const float2 g = s_g[k];
    if (g.x == -INFINITY) continue;        // that chain had no block
    float fa, fb;
    merge_unit_scalars(M, L, g.x, g.y, fa, fb);
    merge4(O, s_o[k * per_row + tid], fa, fb);
  }
  const float inv = 1.0f / L;
  const __nv_bfloat162 a = __floats2bfloat162_rn(O.x * inv, O.y * inv), c = __floats2bfloat162_rn(O.z * inv, O.w * inv);
  *(uint2*)(orow + d4) = make_uint2(*(const uint32_t*)&a, *(const uint32_t*)&c);
}

// One block per (token row, query head): merges the partitions in rising order, normalises, rounds to bf16.
__global__ void attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    const int* __restrict__ seq_row, const int* __restrict__ seg,
                                    __nv_bfloat16* __restrict__ out, int Hq, int HD, int NP, int long_from) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  const int n = blockIdx.y, h = blockIdx.x;
  __nv_bfloat16* orow = out + ((size_t)n * Hq + h) * HD;
  const int row = seq_row[n];
  if (row < 0) {
    for (int d = threadIdx.x; d < HD; d += blockDim.x) orow[d] = __float2bfloat16_rn(0.f);
    return;
  }
  if (seg[row * 4 + 1] >= long_from) return;
  const float* ml = part_ml + ((size_t)n * Hq + h) * NP * 2;
  const float* po = part_o + ((size_t)n * Hq + h) * NP * HD;
  float M = -INFINITY;
  for (int i = 0; i < NP; ++i) M = fmaxf(M, ml[2 * i]);
  float L = 0.f;
  for (int i = 0; i < NP; ++i) L += ml[2 * i + 1] * exp2f(ml[2 * i] - M);
  const float inv = 1.0f / L;
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    float acc = 0.f;
    for (int i = 0; i < NP; ++i) {
      const float f = exp2f(ml[2 * i] - M);
      if (f != 0.f) acc += po[(size_t)i * HD + d] * f;     // an empty partition's O was never written
    }
    orow[d] = __float2bfloat16_rn(acc * inv);
  }
}

template <int HD, int BOX, int NSTAGE, int MINB, bool SMALLG>
int launch_units(const void* q, const void* k_pool, long long pool_rows, const int* pos, const int* seq_row, const int* seg,
                 const int* table, int mb, int page_size, void* out, float* part_o, float* part_ml, int N, int Hq, int Hkv,
                 float scale, int window, int NPU, int long_from, int single, int* err, cudaStream_t stream) {
  CUtensorMap map;
  int st = fztma::get_map_bf16(k_pool, pool_rows, HD, BOX, &map);
  if (st != FZ_OK) return st;
  constexpr size_t stage_bytes = 2 * (HD / 64) * 16 * 128;
  constexpr size_t fixed = 1024 + 4 * NSTAGE * stage_bytes + 8 * 4 * NSTAGE;
  const size_t smem = fixed + (size_t)(N + 1) * 4;
  static int sms = 0;
  static size_t raised = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  if (smem > raised) {
    // (the size grows with the number of rows: raise the limit to the largest the kernel can be asked for)
    const size_t most = fixed + (size_t)(MAX_UNIT_ROWS + 1) * 4;
    cudaError_t e = cudaFuncSetAttribute(attn_decode_units_kernel<HD, BOX, NSTAGE, MINB, SMALLG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most);
    if (e != cudaSuccess) return (int)e;
    raised = most;
  }
  const long long most_units = (long long)N * Hkv * NPU;
  long long ctas = (most_units + 3) / 4;
  if (ctas > (long long)sms * MINB) ctas = (long long)sms * MINB;
  fz_launch(attn_decode_units_kernel<HD, BOX, NSTAGE, MINB, SMALLG>, dim3((unsigned)ctas), dim3(THREADS), smem, stream, map,
            (const __nv_bfloat16*)q, pos, seq_row, seg, table, mb, page_size, part_o, part_ml, N, Hq, Hkv, NPU,
            scale * 1.4426950408889634f, window, long_from, single, err);
  FZ_LAUNCH_CHECK();
  dim3 cgrid(Hq, N);
  // shared memory: the row's (max, sum) pairs, then 256 float4 and up to 16 float2 of the chains' results
  // blocks of 256 threads (a chain per group) while there are fewer blocks than SMs, else of 128 (two chains per group):
  // two engines alternating in one process, a decode step of 32 layers at batch 1 3.100 -> 3.079 ms, batch 2 3.181 ->
  // 3.161, batch 4 3.369 -> 3.348; at batch 8 (256 blocks) 3.780 -> 3.789 and at batch 64 1.3 % slower
  const int ct = (long long)N * Hq <= sms ? 256 : 128;
  fz_launch(attn_combine_units_kernel, cgrid, dim3(ct), (size_t)(NPU + 2) * 8 + 256 * 16 + 16 * 8, stream, (const float*)part_o,
            (const float*)part_ml, pos, seq_row, seg, (__nv_bfloat16*)out, Hq, HD, NPU, window, long_from);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

inline int units_sms() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  return sms;
}
template <int HD, int BOX>
int launch_tma(const void* q, const void* k_pool, long long pool_rows, const int* pos, const int* seq_row, const int* seg,
               const int* table, int mb, int page_size, void* out, float* part_o, float* part_ml, int N, int Hq, int Hkv,
               float scale, int window, int NPU, int long_from, int single, int* err, cudaStream_t stream) {
#define FZ_U(NS_, MB_, SG_) return launch_units<HD, BOX, NS_, MB_, SG_>(q, k_pool, pool_rows, pos, seq_row, seg, table, mb, page_size, out, part_o, part_ml, N, Hq, Hkv, scale, window, NPU, long_from, single, err, stream)
  // three stages of 16 keys per warp and two CTAs per SM (eight warps with 24 KB in flight each) measured best
  if (Hq / Hkv > 8) FZ_U(3, 2, false);
  // So few units that every warp of one CTA per SM gets at most one (a single row at 4,096 keys): four stages, so that
  // a unit's four groups of 16 keys are all asked for at once instead of the fourth waiting for the first to be
  // consumed, one memory round trip later (measured at batch 1: 3.337 -> 3.294 ms per step of 32 layers).
  if ((long long)N * Hkv * NPU <= 4LL * units_sms()) FZ_U(4, 1, true);
  FZ_U(3, 2, true);
#undef FZ_U
}

template <int HD>
int launch(const void* q, const void* k_pool, const void* v_pool, const int* pos, const int* seq_row, const int* seg,
           const int* table, int mb, long long page_stride, int page_size, void* out, float* part_o, float* part_ml,
           int N, int Hq, int Hkv, float scale, int window, int NP, int long_from, cudaStream_t stream) {
  constexpr int TILE_BYTES = TILE * HD * 2;
  constexpr size_t smem_pipe = 2 * STAGES * TILE_BYTES + 16 * HD * 2;
  constexpr size_t smem_merge = (size_t)4 * 16 * (HD + 4) * 4 + 4 * 16 * 2 * 4;
  constexpr size_t smem = smem_pipe > smem_merge ? smem_pipe : smem_merge;
  static bool raised = false;
  if (smem > 48 * 1024 && !raised) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    raised = true;
  }
  dim3 grid(NP, Hkv, N);
  fz_launch(attn_decode_kernel<HD>, grid, dim3(THREADS), smem, stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool,
            (const __nv_bfloat16*)v_pool, pos, seq_row, seg, table, mb, page_stride, page_size, part_o, part_ml, Hq, Hkv,
            scale * 1.4426950408889634f, window, long_from);
  FZ_LAUNCH_CHECK();
  dim3 cgrid(Hq, N);
  fz_launch(attn_combine_kernel, cgrid, dim3(HD < 128 ? 64 : 128), 0, stream, (const float*)part_o, (const float*)part_ml,
            seq_row, seg, (__nv_bfloat16*)out, Hq, HD, NP, long_from);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}
}  // namespace

// Sizes this kernel takes: head_dim 64 or 128, Hq / Hkv <= 16. Anything else is refused (the general kernel takes it).
FZ_API int fz_attn_decode_check(int Hq, int Hkv, int hd) {
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv || Hq / Hkv > 16) return FZ_BAD_SHAPE;
  if (hd != 64 && hd != 128) return FZ_BAD_SHAPE;
  return FZ_OK;
}

// Partial results per (row, head) the scratch must hold for contexts up to max_context: the units of the key axis
// (never fewer than the 256-key partitions of the cp.async variant).
FZ_API int fz_attn_partitions(int max_context) { return max_context <= 0 ? 1 : unit_of(max_context - 1) + 1; }

// Float32 scratch the call needs: part_o N * Hq * NP * hd floats, part_ml N * Hq * NP * 2 floats.
// single_tokens != 0: every portion of the step is one token (the caller knows; the kernel then reads no portion records).
// num_pages > 0 and a pool laid out as (pages, 2, Hkv, page_size, hd) with v_pool = k_pool + Hkv * page_size * hd select
// the TMA variant where the page size allows it (8, 16 or a multiple of 16); otherwise the cp.async variant runs.
FZ_API int fz_attn_decode(const void* q, const void* k_pool, const void* v_pool, const int* pos, const int* seq_row,
                          const int* seg, const int* table, int mb, long long page_stride, int page_size, void* out,
                          float* part_o, float* part_ml, int N, int Hq, int Hkv, int hd, float scale, int window,
                          int max_context, int long_from, int single_tokens, int num_pages, int* err, cudaStream_t stream) {
  if (N <= 0) return FZ_OK;
  const int single = single_tokens ? 1 : 0;
  if (fz_attn_decode_check(Hq, Hkv, hd) != FZ_OK || page_size <= 0) return FZ_BAD_SHAPE;
  if (N > 65535 || Hkv > 65535) return FZ_TOO_LARGE;
  const int NP = max_context <= 0 ? 1 : (max_context + PART - 1) / PART;
  const int NPU = fz_attn_partitions(max_context);
  const bool interleaved = page_stride == 2LL * Hkv * page_size * hd &&
                           (const __nv_bfloat16*)v_pool == (const __nv_bfloat16*)k_pool + (long long)Hkv * page_size * hd;
  const bool tma_ok = num_pages > 0 && interleaved && (((uintptr_t)k_pool) & 15) == 0 &&
                      (page_size == 8 || page_size % 16 == 0) && N <= MAX_UNIT_ROWS &&
                      (long long)N * Hkv * NPU < (1LL << 30) && (size_t)NPU * 8 < 40 * 1024 && !getenv("FZB200_NO_TMA_ATTN");
  if (tma_ok) {
    const long long pool_rows = (long long)num_pages * 2 * Hkv * page_size;
#define FZ_T(HD_, BOX_) return launch_tma<HD_, BOX_>(q, k_pool, pool_rows, pos, seq_row, seg, table, mb, page_size, out, part_o, part_ml, N, Hq, Hkv, scale, window, NPU, long_from, single, err, stream)
    if (hd == 64 && page_size == 8) FZ_T(64, 8);
    if (hd == 64) FZ_T(64, 16);
    if (page_size == 8) FZ_T(128, 8);
    FZ_T(128, 16);
#undef FZ_T
  }
  if (hd == 64)
    return launch<64>(q, k_pool, v_pool, pos, seq_row, seg, table, mb, page_stride, page_size, out, part_o, part_ml, N, Hq, Hkv, scale, window, NP, long_from, stream);
  return launch<128>(q, k_pool, v_pool, pos, seq_row, seg, table, mb, page_stride, page_size, out, part_o, part_ml, N, Hq, Hkv, scale, window, NP, long_from, stream);
}

#ifdef FZ_TIMELINE
FZ_TIMELINE_READER(attn_decode)
#endif
