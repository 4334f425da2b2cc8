// Causal flash attention for prompt portions over the paged bf16 cache on the 5th-generation tensor cores.
//
// grid (tiles, query heads), 352 threads, one CTA per SM. A tile is 128 consecutive token rows of one portion (the host
// lists the tiles, the ones with the most keys first); the 128 rows are the 128 TMEM lanes. Keys come in tiles of 128:
//   warps 0, 10 TMA producers: warp 0 the Q tile once and the key tiles, warp 10 the value tiles (a page's rows of one kv
//               head are one box of the pool seen as a 2-D array of rows; 128-byte swizzle), each into a ring of its own
//               and as far ahead as the ring allows (a key stage is free again as soon as its score product is done);
//   warp 1      one lane issues tcgen05.mma: S = Q K^T (128 x 128 x hd, both operands K-major) into one of two TMEM
//               buffers, one key tile ahead of the softmax warps, and, once they have written P, PV = P V (128 x hd x
//               128; V is the MN-major operand, as TMA delivers it) into one of two more;
//   warps 2..9  two threads per row, each with 64 of the tile's 128 score columns and half of the output dimensions (the
//               two warps of a row pair sit on one scheduler, so one computes while the other waits): read the
//               scores from TMEM once, scale, mask (causal by position, window), exchange the row maximum through
//               shared memory, online softmax in the exp2 domain with float32 max and sum, write P as bf16 into one of
//               two shared-memory buffers in the swizzled K-major layout; then fold the PV product of the tile
//               *before* into the float32 output registers, so that the tensor core computes a tile's PV while
//               these warps already work on the next tile's scores. At the end normalise and store the row.
// Key tiles start at multiples of 128 in absolute position, so a row's sums do not depend on how the prompt was cut.
// Waits on the CTA's own mbarriers are bounded; a wait that gives up sets the error bit. No multicast.
// (The reference's paged prefill kernel is an mma.sync kernel with 64-row tiles: fusezap/device/cuda_kernels/
// attention.py:255-326; `attn_prefill.cu` here is its counterpart and serves the page sizes this kernel refuses.)
#include "umma.cuh"
#include <math.h>

namespace {
using namespace fztma;
using namespace fzumma;

constexpr int BM = 128, BN = 128, NUM_THREADS = 352;

template <int HD, int BOX>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map,
                       const int* __restrict__ seg, const int* __restrict__ tiles, const int* __restrict__ table, int mb,
                       int page_size, __nv_bfloat16* __restrict__ out, int Hq, int Hkv, float scale_log2, int window,
                       int* err) {
  constexpr int HALVES = HD / 64;                     // 64-column halves of a head
  constexpr int KV_STAGES = HD <= 64 ? 4 : 2;         // key tiles and value tiles in flight (what shared memory holds)
  constexpr int HALF_BYTES = 128 * 128;               // 128 rows of 128 bytes
  constexpr int Q_BYTES = HALVES * HALF_BYTES, KV_BYTES = HALVES * HALF_BYTES, P_BYTES = (BN / 64) * HALF_BYTES;
  constexpr int TMEM_COLS = 512;                      // S: columns 0..127 and 128..255; PV: 256.. and 384..
  constexpr int OPS = (BN / BOX) * HALVES;            // TMA boxes per key tile, for K and again for V
  constexpr int OD = HD / 2;                          // output dimensions per thread
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  // [Q][K ring][V ring][P x 2][row maxima][barriers]
  const uint32_t s_q = smem_u32(smem), s_k = s_q + Q_BYTES, s_v = s_k + KV_STAGES * KV_BYTES, s_p = s_v + KV_STAGES * KV_BYTES;
  float* s_mx = (float*)(smem + Q_BYTES + 2 * KV_STAGES * KV_BYTES + 2 * P_BYTES);      // [2 halves][128 rows]
  uint64_t* bars = (uint64_t*)(s_mx + 2 * BM);
  uint64_t* q_full = bars;                 // 1
  uint64_t* k_full = bars + 1;             // KV_STAGES each
  uint64_t* k_empty = k_full + KV_STAGES;
  uint64_t* v_full = k_empty + KV_STAGES;
  uint64_t* v_empty = v_full + KV_STAGES;
  uint64_t* s_ready = v_empty + KV_STAGES; // 2: one per S buffer
  uint64_t* p_ready = s_ready + 2;         // 2: one per P buffer
  uint64_t* pv_ready = p_ready + 2;        // 2: one per PV buffer
  uint64_t* pv_free = pv_ready + 2;        // 2
  uint32_t* tmem_slot = (uint32_t*)(pv_free + 2);
  int* flag = (int*)(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_ready[i], 1);
      mbar_init(&p_ready[i], 256);
      mbar_init(&pv_ready[i], 1);
      mbar_init(&pv_free[i], 256);
    }
    flag[0] = 0;
    mbar_init_fence();
  }
  // zeros in the key / value stages: a box that is not fetched (keys past the portion's last position) must not hold
  // another block's bits, since P = 0 times NaN is NaN
  for (int e = tid; e < 2 * KV_STAGES * KV_BYTES / 16; e += NUM_THREADS) ((uint4*)(smem + Q_BYTES))[e] = make_uint4(0u, 0u, 0u, 0u);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  fz_grid_launch_dependents();
  // (the tile list, the portions and the block tables are the step's metadata: written by the host before the step's
  // first kernel, so they may be read ahead of the wait on the kernel before this one)
  const int s_idx = tiles[2 * blockIdx.x], r_off = tiles[2 * blockIdx.x + 1];
  const int h = blockIdx.y, kvh = h / (Hq / Hkv);
  int n_key_tiles = 0, row0 = 0, valid_rows = 0, qpos0 = 0, last_pos = 0, lo_tile = 0, k_begin = 0;
  if (s_idx >= 0) {
    row0 = seg[4 * s_idx];
    const int n_rows = seg[4 * s_idx + 1], pos0 = seg[4 * s_idx + 2];
    valid_rows = min(BM, n_rows - r_off);
    qpos0 = pos0 + r_off;
    last_pos = qpos0 + valid_rows - 1;
    lo_tile = window > 0 ? max(0, qpos0 - window + 1) : 0;
    k_begin = lo_tile & ~(BN - 1);
    n_key_tiles = (last_pos - k_begin) / BN + 1;
  }
  fz_grid_wait();

  if (warp == 0 || warp == 10) {
    // ---------------- TMA producers: warp 0 the Q tile and the key tiles, warp 10 the value tiles; each runs as far
    // ahead as its ring allows (a key stage is free once its score product is done, a value stage once its PV is)
    const bool is_v = warp == 10;
    if (n_key_tiles > 0) {
      if (!is_v && lane == 0) {
        mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
        for (int hf = 0; hf < HALVES; ++hf) tma_load_2d_u32(s_q + hf * HALF_BYTES, &q_map, smem_u32(q_full), h * HD + 64 * hf, row0 + r_off);
      }
      const int* trow = table + (size_t)s_idx * mb;
      const int rows_per_page = 2 * Hkv * page_size;
      bool ok = true;
      for (int t = 0; t < n_key_tiles && ok; ++t) {
        const int s = t % KV_STAGES, round = t / KV_STAGES;
        const int key0 = k_begin + t * BN;
        // op -> (page box, column half); a box is fetched if any of its keys lies in [lo_tile, last_pos]
        int op_row[(OPS + 31) / 32];
        uint32_t bytes = 0;
#pragma unroll
        for (int i = 0; i < (OPS + 31) / 32; ++i) {
          const int op = lane + 32 * i;
          op_row[i] = -1;
          if (op < OPS) {
            const int box = op / HALVES;
            const int key = key0 + box * BOX;
            if (key <= last_pos && key + BOX - 1 >= lo_tile) {
              const int pi = key / page_size;
              const int page = trow[pi];
              if (page >= 0) op_row[i] = page * rows_per_page + kvh * page_size + (key - pi * page_size);
              else if (!is_v) atomicOr(err, FZ_ERR_NO_PAGE);
            }
          }
          bytes += op_row[i] >= 0 ? BOX * 128u : 0u;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) bytes += __shfl_xor_sync(0xffffffffu, bytes, o);
        uint64_t* full = is_v ? &v_full[s] : &k_full[s];
        uint64_t* empty = is_v ? &v_empty[s] : &k_empty[s];
        if (round > 0) ok = __all_sync(0xffffffffu, mbar_wait(empty, (round - 1) & 1));
        if (!ok) break;
        if (lane == 0) mbar_expect_tx(full, bytes);
        __syncwarp();
        const uint32_t dst = (is_v ? s_v : s_k) + s * KV_BYTES, bar = smem_u32(full);
#pragma unroll
        for (int i = 0; i < (OPS + 31) / 32; ++i) {
          const int op = lane + 32 * i;
          if (op < OPS && op_row[i] >= 0) {
            const int box = op / HALVES, hf = op % HALVES;
            tma_load_2d_u32(dst + hf * HALF_BYTES + box * BOX * 128, &kv_map, bar, 64 * hf, op_row[i] + (is_v ? Hkv * page_size : 0));
          }
        }
      }
      if (!ok && lane == 0) flag[0] = 1;
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer
    if (lane == 0 && n_key_tiles > 0) {
      constexpr uint32_t idesc_s = make_idesc(BM, BN, false), idesc_pv = make_idesc(BM, HD, true);
      bool ok = mbar_wait(q_full, 0);
      auto issue_s = [&](int t) -> bool {      // S(t) = Q K(t)^T into S buffer t & 1; frees the key stage when done
        const int s = t % KV_STAGES;
        if (!mbar_wait(&k_full[s], (t / KV_STAGES) & 1)) return false;
        tc_fence_after();
        const uint32_t sk = s_k + s * KV_BYTES, tmem_s = tmem_base + (uint32_t)(t & 1) * 128u;
#pragma unroll
        for (int hf = 0; hf < HALVES; ++hf) {
          const uint64_t dq = desc_k_major(s_q + hf * HALF_BYTES), dk = desc_k_major(sk + hf * HALF_BYTES);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_bf16(tmem_s, dq + (uint64_t)(2 * k), dk + (uint64_t)(2 * k), idesc_s, (hf | k) ? 1u : 0u);
        }
        umma_commit(&s_ready[t & 1]);
        umma_commit(&k_empty[s]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int t = 0; t < n_key_tiles && ok; ++t) {
        // the next tile's scores run on the tensor core while the softmax warps work on this tile's
        if (t + 1 < n_key_tiles && !issue_s(t + 1)) { ok = false; break; }
        const int s = t % KV_STAGES, b = t & 1;
        if (!mbar_wait(&v_full[s], (t / KV_STAGES) & 1)) { ok = false; break; }
        if (!mbar_wait(&p_ready[b], (t >> 1) & 1)) { ok = false; break; }
        if (t >= 2 && !mbar_wait(&pv_free[b], ((t >> 1) - 1) & 1)) { ok = false; break; }   // PV(t - 2) has been folded
        tc_fence_after();
        const uint32_t sv = s_v + s * KV_BYTES, sp = s_p + b * P_BYTES, tmem_pv = tmem_base + 256u + (uint32_t)b * 128u;
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const uint64_t dp = desc_k_major(sp + (kk >> 2) * HALF_BYTES) + (uint64_t)(2 * (kk & 3));
          const uint64_t dv = desc_mn_major(sv + kk * 16 * 128, HALF_BYTES);
          umma_bf16(tmem_pv, dp, dv, idesc_pv, kk ? 1u : 0u);
        }
        umma_commit(&pv_ready[b]);
        umma_commit(&v_empty[s]);
      }
      if (!ok) flag[0] = 1;
    }
  } else {
    // ---------------- softmax and output: two threads per row
    const int quad = warp & 3, hf = (warp - 2) >> 2;          // warps w and w + 4 share the row quarter `quad`
    const int r = quad * 32 + lane;
    const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
    const int qpos = qpos0 + r;
    const int pair_bar = 1 + quad;                             // named barrier of the two warps of this row quarter
    float o[OD];
#pragma unroll
    for (int i = 0; i < OD; ++i) o[i] = 0.f;
    float m_run = -INFINITY, l_part = 0.f, corr_pending = 1.f;
    bool ok = true;
    auto fold = [&](int t) -> bool {      // o = o * (rescale of tile t) + PV(t), this thread's half of the dimensions
      const int b = t & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&pv_ready[b], (t >> 1) & 1))) return false;
      tc_fence_after();
      const uint32_t t_pv = tmem_base + 256u + (uint32_t)b * 128u + (uint32_t)(hf * OD) + lane_sel;
      float v[32];
#pragma unroll
      for (int c = 0; c < OD; c += 32) {
        tmem_ld32(t_pv + (uint32_t)c, v);
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c + i] = fmaf(o[c + i], corr_pending, v[i]);
      }
      tc_fence_before();
      mbar_arrive(&pv_free[b]);
      return true;
    };
    for (int t = 0; t < n_key_tiles && ok; ++t) {
      const int b = t & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&s_ready[b], (t >> 1) & 1));
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_s = tmem_base + (uint32_t)b * 128u + (uint32_t)(hf * 64) + lane_sel;
      const int key0 = k_begin + t * BN + hf * 64;
      const int lo_key = window > 0 ? max(lo_tile, qpos - window + 1) : lo_tile;
      const bool full = key0 + 63 <= qpos && key0 >= lo_key;     // every key of this thread's half is visible to its row
      float v[64];
      tmem_ld32(t_s, v);
      tmem_ld32(t_s + 32u, v + 32);
      if (!full) {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const int key = key0 + i;
          v[i] = (key <= qpos && key >= lo_key) ? v[i] : -INFINITY;      // exp2(-inf) = 0 below
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};       // four chains, so that the maxima do not wait on one another
#pragma unroll
      for (int i = 0; i < 64; i += 4) {
        mx4[0] = fmaxf(mx4[0], v[i]); mx4[1] = fmaxf(mx4[1], v[i + 1]); mx4[2] = fmaxf(mx4[2], v[i + 2]); mx4[3] = fmaxf(mx4[3], v[i + 3]);
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // the row's maximum over both halves
      s_mx[hf * BM + r] = mx;
      asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
      mx = fmaxf(mx, s_mx[(hf ^ 1) * BM + r]);
      asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");    // both have read: the slots may be written again
      const float mn = fmaxf(m_run, mx * scale_log2);
      const float mu = mn == -INFINITY ? 0.f : mn;
      const float corr = fast_exp2(m_run - mu);
      m_run = mn;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};      // four chains again; added up in a fixed order below
      // this thread's 64 columns of row r: column half hf, 16-byte chunks 0..7, swizzled by the row
      const uint32_t base = s_p + b * P_BYTES + hf * HALF_BYTES + r * 128;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float e0 = fast_exp2(fmaf(v[8 * j + 2 * i], scale_log2, -mu)), e1 = fast_exp2(fmaf(v[8 * j + 2 * i + 1], scale_log2, -mu));
          sum4[i] += e0 + e1;
          const __nv_bfloat162 pk = __floats2bfloat162_rn(e0, e1);
          w[i] = *(const uint32_t*)&pk;
        }
        const uint32_t addr = base + ((j ^ (r & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
      }
      l_part = l_part * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P is read by the tensor core (async proxy)
      tc_fence_before();
      mbar_arrive(&p_ready[b]);
      if (t > 0) ok = fold(t - 1);      // the tile before: its PV ran while this tile's scores were worked on
      corr_pending = corr;
    }
    if (ok && n_key_tiles > 0) ok = fold(n_key_tiles - 1);
    if (!ok) flag[0] = 1;
    // the row's sum of weights: half 0 + half 1
    s_mx[hf * BM + r] = l_part;
    asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
    const float l_run = s_mx[r] + s_mx[BM + r];
    if (ok && n_key_tiles > 0 && r < valid_rows) {
      const float inv = 1.0f / l_run;
      __nv_bfloat16* orow = out + (size_t)(row0 + r_off + r) * Hq * HD + (size_t)h * HD + hf * OD;
#pragma unroll
      for (int c = 0; c < OD; c += 8) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const __nv_bfloat162 pk = __floats2bfloat162_rn(o[c + 2 * j] * inv, o[c + 2 * j + 1] * inv);
          w[j] = *(const uint32_t*)&pk;
        }
        *(uint4*)(orow + c) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (tid == 0 && flag[0]) atomicOr(err, FZ_ERR_WAIT_TIMEOUT);
}

template <int HD, int BOX>
int launch(const void* q, int N, const void* k_pool, long long pool_rows, const int* seg, const int* tiles, int n_tiles,
           const int* table, int mb, int page_size, void* out, int Hq, int Hkv, float scale, int window, int* err,
           cudaStream_t stream) {
  CUtensorMap qm, kvm;
  int st = get_map_bf16(q, N, Hq * HD, BM, &qm);
  if (st != FZ_OK) return st;
  if ((st = get_map_bf16(k_pool, pool_rows, HD, BOX, &kvm)) != FZ_OK) return st;
  constexpr int HALVES = HD / 64, HALF_BYTES = 128 * 128;
  constexpr int KV_STAGES = HD <= 64 ? 4 : 2;
  constexpr size_t smem = (size_t)HALVES * HALF_BYTES + KV_STAGES * 2 * HALVES * HALF_BYTES + 2 * (BN / 64) * HALF_BYTES + 2 * BM * 4 + 8 * 32 + 1024;
  static bool raised = false;
  if (!raised) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<HD, BOX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    raised = true;
  }
  dim3 grid(n_tiles, Hq);
  fz_launch(attn_prefill_tc_kernel<HD, BOX>, grid, dim3(NUM_THREADS), smem, stream, qm, kvm, seg, tiles, table, mb, page_size,
            (__nv_bfloat16*)out, Hq, Hkv, scale * 1.4426950408889634f, window, err);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}
}  // namespace

// Takes head sizes 64 and 128 and page sizes 8, 16 and multiples of 16, with the pool laid out as (pages, 2, Hkv,
// page_size, hd); anything else is refused and the mma.sync kernel runs instead.
FZ_API int fz_attn_prefill_tc_check(int Hq, int Hkv, int hd, int page_size) {
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv) return FZ_BAD_SHAPE;
  if (hd != 64 && hd != 128) return FZ_BAD_SHAPE;
  if (!(page_size == 8 || (page_size > 0 && page_size % 16 == 0))) return FZ_BAD_SHAPE;
  return FZ_OK;
}

// tiles: int32 [n_tiles][2] = (portion index or -1, first row of the 128-row tile within the portion). q: [N, Hq * hd].
FZ_API int fz_attn_prefill_tc(const void* q, int N, const void* k_pool, const void* v_pool, long long page_stride,
                              int num_pages, const int* seg, const int* tiles, int n_tiles, const int* table, int mb,
                              int page_size, void* out, int Hq, int Hkv, int hd, float scale, int window, int* err,
                              cudaStream_t stream) {
  if (n_tiles <= 0) return FZ_OK;
  if (fz_attn_prefill_tc_check(Hq, Hkv, hd, page_size) != FZ_OK || Hq > 65535) return FZ_BAD_SHAPE;
  if (page_stride != 2LL * Hkv * page_size * hd ||
      (const __nv_bfloat16*)v_pool != (const __nv_bfloat16*)k_pool + (long long)Hkv * page_size * hd)
    return FZ_BAD_SHAPE;
  if ((((uintptr_t)q) | ((uintptr_t)k_pool) | ((uintptr_t)out)) & 15) return FZ_BAD_ALIGNMENT;
  const long long pool_rows = (long long)num_pages * 2 * Hkv * page_size;
#define FZ_T(HD_, BOX_) return launch<HD_, BOX_>(q, N, k_pool, pool_rows, seg, tiles, n_tiles, table, mb, page_size, out, Hq, Hkv, scale, window, err, stream)
  // the largest box a page allows: a key tile of 128 keys is then 2, 8 or 16 boxes per column half
  if (hd == 64 && page_size == 8) FZ_T(64, 8);
  if (hd == 64 && page_size % 64 == 0) FZ_T(64, 64);
  if (hd == 64) FZ_T(64, 16);
  if (page_size == 8) FZ_T(128, 8);
  if (page_size % 64 == 0) FZ_T(128, 64);
  FZ_T(128, 16);
#undef FZ_T
}
