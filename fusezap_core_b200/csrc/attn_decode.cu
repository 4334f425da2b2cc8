// Paged attention for decoded tokens and short portions, bf16 cache, on tensor cores, split over key partitions.
//
// grid (partitions, kv heads, token rows), 128 threads. A CTA serves one token row, one kv head and one partition of
// PART = 256 consecutive key positions (partition i holds keys 256 i .. 256 i + 255, whatever the batch: a row's sums
// have one order that depends only on its own position). All G = Hq / Hkv query heads of the kv head are the rows of
// the 16-row MMA tile, so the keys and values of the partition are read once for the whole group (the reference's
// default decode kernel lays the group out the same way: fusezap/device/cuda_kernels/attention.py:860-1043).
// Keys and values come in tiles of 64 through a three-stage cp.async ring; warp w owns keys 16 w .. 16 w + 15 of each
// tile: S = Q K^T and O += P V with mma.sync m16n8k16, softmax online in the exp2 domain with float32 max and sum, P
// rounded to bf16 for the second product. The four warps' (max, sum, O) are merged in warp order, and the partition's
// unnormalised O with its (max, sum) goes to a float32 scratch; `attn_combine_kernel` merges a row's partitions in
// rising order and normalises. Rows of portions with at least `long_from` tokens are left to the prefill kernel.
//
// Two variants load the keys and values. `attn_decode_tma_kernel` (page sizes 8, 16 and multiples of 16): every warp
// fetches its own 16-key groups with TMA tile loads (a page's rows of one kv head are one box of the pool seen as a
// 2-D array of rows; 128-byte swizzle) into a two-deep ring of its own, guarded by mbarriers, with no block-wide
// barrier in the loop; this is what keeps enough bytes in flight for HBM3e. `attn_decode_kernel` (any page size)
// gathers 64-key tiles with cp.async through a three-stage ring.
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
  fz_grid_wait();
  fz_grid_launch_dependents();
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
// kv_map: the cache slot's pool seen as a row-major [pages * 2 * Hkv * page_size, HD] bf16 array (row of key `off` of kv
// head `kvh` of page `pg`: pg * 2 Hkv bs + kvh * bs + off; its value row: + Hkv * bs), boxes of BOX rows x 64 columns.
// Shared memory per warp: 2 stages x [K | V], each HD / 64 column halves of [16 rows][128 bytes], swizzled by TMA.
constexpr int TMA_DEPTH = 2;

template <int HD, int BOX>
__global__ void __launch_bounds__(THREADS)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap kv_map, const __nv_bfloat16* __restrict__ q,
                       const int* __restrict__ pos, const int* __restrict__ seq_row, const int* __restrict__ seg,
                       const int* __restrict__ table, int mb, int page_size, float* __restrict__ part_o,
                       float* __restrict__ part_ml, int Hq, int Hkv, float scale_log2, int window, int long_from,
                       int* err) {
  constexpr int KSTEPS = HD / 16, NB = HD / 8, HALVES = HD / 64;
  constexpr int HALF_BYTES = 16 * 128;                 // one column half of a 16-key group
  constexpr int KV_BYTES = HALVES * HALF_BYTES;        // keys (or values) of a group
  constexpr int STAGE_BYTES = 2 * KV_BYTES;
  constexpr int WARP_BYTES = TMA_DEPTH * STAGE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t s_base = smem_u32(smem);
  const uint32_t s_q = s_base + 4 * WARP_BYTES;
  uint64_t* bars = (uint64_t*)(smem + 4 * WARP_BYTES + 16 * HD * 2);    // [4 warps][TMA_DEPTH]

  // Prologue that depends on nothing another kernel writes: barriers, and zeros in the staging buffers (a box that is
  // not fetched because it lies past the row's position must not hold another block's bits: P = 0 times NaN is NaN).
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int i = 0; i < 4 * TMA_DEPTH; ++i) fztma::mbar_init(&bars[i], 1);
    fztma::mbar_init_fence();
  }
  for (int e = tid; e < 4 * WARP_BYTES / 16; e += THREADS) ((uint4*)smem)[e] = make_uint4(0u, 0u, 0u, 0u);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  fz_grid_wait();
  fz_grid_launch_dependents();

  const int part = blockIdx.x, kvh = blockIdx.y, n = blockIdx.z, NP = gridDim.x;
  const int G = Hq / Hkv;
  const int row = seq_row[n];
  if (row < 0) return;
  if (seg[row * 4 + 1] >= long_from) return;
  const int p = pos[n];
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int k_begin = max(part * PART, lo & ~(TILE - 1)), k_end = min((part + 1) * PART, p + 1);
  float* ml_out = part_ml + (((size_t)n * Hq + (size_t)kvh * G) * NP + part) * 2;
  if (k_begin >= k_end) {
    for (int g = tid; g < G; g += THREADS) { ml_out[(size_t)g * NP * 2] = -INFINITY; ml_out[(size_t)g * NP * 2 + 1] = 0.f; }
    return;
  }
  const int* trow = table + (size_t)row * mb;
  const int rows_per_page = 2 * Hkv * page_size;
  {
    const __nv_bfloat16* qrow = q + (size_t)n * Hq * HD + (size_t)kvh * G * HD;
    for (int e = tid; e < 16 * (HD / 8); e += THREADS) {
      const int r = e / (HD / 8), c = e - r * (HD / 8);
      cp_async16(s_q + swz<HD>(r, c), qrow + (size_t)r * HD + c * 8, r < G);
    }
    cp_async_commit();
  }
  // this warp's groups of 16 keys: group g holds keys k_begin + 16 g .., g = warp, warp + 4, ...
  const int n_groups = (k_end - k_begin + 15) / 16;
  const int my_groups = n_groups > warp ? (n_groups - warp + 3) / 4 : 0;
  const uint32_t s_warp = s_base + warp * WARP_BYTES;
  auto issue = [&](int j) {        // lane 0 only
    const int stage = j % TMA_DEPTH;
    const int key0 = k_begin + 16 * (warp + 4 * j);
    uint64_t* bar = &bars[warp * TMA_DEPTH + stage];
    int rows[16 / BOX];
    uint32_t bytes = 0;
#pragma unroll
    for (int sub = 0; sub < 16 / BOX; ++sub) {
      const int key = key0 + sub * BOX;
      rows[sub] = -1;
      if (key > p || key + BOX - 1 < lo) continue;       // nothing visible in this box
      const int pi = key / page_size;
      const int page = trow[pi];
      if (page < 0) { atomicOr(err, FZ_ERR_NO_PAGE); continue; }
      rows[sub] = page * rows_per_page + kvh * page_size + (key - pi * page_size);
      bytes += 2 * HALVES * BOX * 128;
    }
    fztma::mbar_expect_tx(bar, bytes);
    const uint32_t sk = s_warp + stage * STAGE_BYTES, sv = sk + KV_BYTES, b = smem_u32(bar);
#pragma unroll
    for (int sub = 0; sub < 16 / BOX; ++sub) {
      if (rows[sub] < 0) continue;
#pragma unroll
      for (int h = 0; h < HALVES; ++h) {
        fztma::tma_load_2d_u32(sk + h * HALF_BYTES + sub * BOX * 128, &kv_map, b, 64 * h, rows[sub]);
        fztma::tma_load_2d_u32(sv + h * HALF_BYTES + sub * BOX * 128, &kv_map, b, 64 * h, rows[sub] + Hkv * page_size);
      }
    }
  };
  if (lane == 0) {
#pragma unroll
    for (int j = 0; j < TMA_DEPTH; ++j)
      if (j < my_groups) issue(j);
  }
  cp_async_wait<0>();
  __syncthreads();
  uint32_t qf[KSTEPS][4];
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) ldmatrix_x4(qf[ks], s_q + swz<HD>(lane & 15, ks * 2 + (lane >> 4)));
  float o[NB][4];
#pragma unroll
  for (int i = 0; i < NB; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  bool timed_out = false;
  for (int j = 0; j < my_groups; ++j) {
    const int stage = j % TMA_DEPTH;
    if (!__all_sync(0xffffffffu, fztma::mbar_wait(&bars[warp * TMA_DEPTH + stage], (j / TMA_DEPTH) & 1))) { timed_out = true; break; }
    const uint32_t sk = s_warp + stage * STAGE_BYTES, sv = sk + KV_BYTES;
    // chunk c of row r: column half c >> 3, 16-byte chunk (c & 7) ^ (r & 7) of the 128-byte row (TMA's swizzle)
    attend16<HD>(qf, [&](int r, int c) { return sk + (c >> 3) * HALF_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4); },
                 [&](int r, int c) { return sv + (c >> 3) * HALF_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4); },
                 k_begin + 16 * (warp + 4 * j), lo, p, scale_log2, o, m_run, l_run, lane);
    __syncwarp();
    if (lane == 0 && j + TMA_DEPTH < my_groups) issue(j + TMA_DEPTH);
  }
  if (timed_out && lane == 0) atomicOr(err, FZ_ERR_WAIT_TIMEOUT);
  __syncthreads();     // every warp has consumed all it requested: the staging buffers are free for the merge
  merge_and_store<HD>((float*)smem, o, m_run, l_run, part_o, ml_out, n, Hq, kvh, G, NP, part, tid);
}

// One block per (token row, query head): merges the partitions in rising order, normalises, rounds to bf16.
__global__ void attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    const int* __restrict__ seq_row, const int* __restrict__ seg,
                                    __nv_bfloat16* __restrict__ out, int Hq, int HD, int NP, int long_from) {
  fz_grid_wait();
  fz_grid_launch_dependents();
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

template <int HD, int BOX>
int launch_tma(const void* q, const void* k_pool, long long pool_rows, const int* pos, const int* seq_row, const int* seg,
               const int* table, int mb, int page_size, void* out, float* part_o, float* part_ml, int N, int Hq, int Hkv,
               float scale, int window, int NP, int long_from, int* err, cudaStream_t stream) {
  CUtensorMap map;
  int st = fztma::get_map_bf16(k_pool, pool_rows, HD, BOX, &map);
  if (st != FZ_OK) return st;
  constexpr size_t stage_bytes = 2 * (HD / 64) * 16 * 128;
  constexpr size_t smem_pipe = 4 * TMA_DEPTH * stage_bytes + 16 * HD * 2 + 8 * 4 * TMA_DEPTH;
  constexpr size_t smem_merge = (size_t)4 * 16 * (HD + 4) * 4 + 4 * 16 * 2 * 4;
  constexpr size_t smem = (smem_pipe > smem_merge ? smem_pipe : smem_merge) + 1024;
  static bool raised = false;
  if (smem > 48 * 1024 && !raised) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_tma_kernel<HD, BOX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    raised = true;
  }
  dim3 grid(NP, Hkv, N);
  fz_launch(attn_decode_tma_kernel<HD, BOX>, grid, dim3(THREADS), smem, stream, map, (const __nv_bfloat16*)q, pos, seq_row, seg,
            table, mb, page_size, part_o, part_ml, Hq, Hkv, scale * 1.4426950408889634f, window, long_from, err);
  FZ_LAUNCH_CHECK();
  dim3 cgrid(Hq, N);
  fz_launch(attn_combine_kernel, cgrid, dim3(HD < 128 ? 64 : 128), 0, stream, (const float*)part_o, (const float*)part_ml,
            seq_row, seg, (__nv_bfloat16*)out, Hq, HD, NP, long_from);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
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

FZ_API int fz_attn_partitions(int max_context) { return max_context <= 0 ? 1 : (max_context + PART - 1) / PART; }

// Float32 scratch the call needs: part_o N * Hq * NP * hd floats, part_ml N * Hq * NP * 2 floats.
// num_pages > 0 and a pool laid out as (pages, 2, Hkv, page_size, hd) with v_pool = k_pool + Hkv * page_size * hd select
// the TMA variant where the page size allows it (8, 16 or a multiple of 16); otherwise the cp.async variant runs.
FZ_API int fz_attn_decode(const void* q, const void* k_pool, const void* v_pool, const int* pos, const int* seq_row,
                          const int* seg, const int* table, int mb, long long page_stride, int page_size, void* out,
                          float* part_o, float* part_ml, int N, int Hq, int Hkv, int hd, float scale, int window,
                          int max_context, int long_from, int num_pages, int* err, cudaStream_t stream) {
  if (N <= 0) return FZ_OK;
  if (fz_attn_decode_check(Hq, Hkv, hd) != FZ_OK || page_size <= 0) return FZ_BAD_SHAPE;
  if (N > 65535 || Hkv > 65535) return FZ_TOO_LARGE;
  const int NP = fz_attn_partitions(max_context);
  const bool interleaved = page_stride == 2LL * Hkv * page_size * hd &&
                           (const __nv_bfloat16*)v_pool == (const __nv_bfloat16*)k_pool + (long long)Hkv * page_size * hd;
  const bool tma_ok = num_pages > 0 && interleaved && (((uintptr_t)k_pool) & 15) == 0 &&
                      (page_size == 8 || page_size % 16 == 0) && !getenv("FZB200_NO_TMA_ATTN");
  if (tma_ok) {
    const long long pool_rows = (long long)num_pages * 2 * Hkv * page_size;
#define FZ_T(HD_, BOX_) return launch_tma<HD_, BOX_>(q, k_pool, pool_rows, pos, seq_row, seg, table, mb, page_size, out, part_o, part_ml, N, Hq, Hkv, scale, window, NP, long_from, err, stream)
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
