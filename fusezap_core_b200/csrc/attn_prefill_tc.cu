// Causal flash attention for prompt portions over the paged bf16 cache on the 5th-generation tensor cores.
//
// One block per SM (352 threads), each walking its share of the work items: an item is a tile of 128 consecutive token
// rows of one portion (the host lists the tiles, the ones with the most keys first) and one query head; items are dealt
// out in rows of gridDim.x, every other row backwards, which evens out the causal tile sizes. The 128 rows are the 128
// TMEM lanes. Keys come in tiles of 128; every role counts the key tiles it has gone through, so rings, buffers and
// barrier phases carry over from item to item and the producers fetch the next item's tiles while this one finishes:
//   warps 0, 10 TMA producers: warp 0 the Q tile (once the last score product of the item before has freed it) and the
//               key tiles, warp 10 the value tiles (a page's rows of one kv head are one box of the pool seen as a 2-D
//               array of rows; 128-byte swizzle), each into a ring of its own and as far ahead as the ring allows (a
//               key stage is free again as soon as its score product is done);
//   warp 1      one lane issues tcgen05.mma: S = Q K^T (128 x 128 x hd, both operands K-major) into one of two TMEM
//               buffers, one key tile ahead of the softmax warps, and, once they have written P, O += P V (128 x hd x
//               128; P is the A operand in tensor memory, V the MN-major B operand as TMA delivers it), accumulated in
//               tensor memory over the item's key tiles;
//   warps 2..9  two threads per row, each with 64 of the tile's 128 score columns and half of the output dimensions (the
//               two warps of a row pair sit on one scheduler, so one computes while the other waits): read the
//               scores from TMEM once, scale, mask (causal by position, window), exchange the row maximum through
//               shared memory, online softmax in the exp2 domain with float32 max and sum (packed float32 x 2
//               arithmetic; three pairs of exponentials in eight by a polynomial on the FMA pipe, the rest on the
//               special-function unit), write P as bf16 pairs back into tensor memory over the scores they came from.
//               O stays in tensor memory and is rescaled there only when a row's maximum has grown by more than 2^8
//               over the maximum in use, so it costs no registers; at the item's end normalise and store the rows.
// Key tiles start at multiples of 128 in absolute position, so a row's sums do not depend on how the prompt was cut.
// `attn_prefill_pair_kernel` is the same with two query heads of one kv head per block (608 threads: each head its own
// score / P and output columns and eight softmax warps, one MMA lane alternating between them, key and value stages
// fetched once for both). An entry of the host's list may be a PIECE of a query tile along the keys (a small portion
// behind a long prefix would otherwise leave most SMs idle): its items leave unnormalised rows in float32 scratch and
// `attn_prefill_merge_kernel` adds a tile's pieces up in entry order.
// Waits on the CTA's own mbarriers are bounded; a wait that gives up sets the error bit. No multicast.
// (The reference's paged prefill kernel is an mma.sync kernel with 64-row tiles: fusezap/device/cuda_kernels/
// attention.py:255-326; `attn_prefill.cu` here is its counterpart and serves the page sizes this kernel refuses.)
#include "umma.cuh"
#include <math.h>

namespace {
using namespace fztma;
using namespace fzumma;

constexpr int BM = 128, BN = 128, NUM_THREADS = 352;
constexpr int PAIR_THREADS = 608;       // the two-tile kernel: TMA, MMA, 16 softmax warps, TMA
constexpr float RESCALE_STEP = 8.f;

// One work item: a 128-row tile of a portion and one query head.
struct Item {
  int n_key_tiles, s_idx, h, row, valid_rows, qpos0, last_pos, lo_tile, k_begin, slot;
};

// An entry of the host's list is (portion or -1, first row of the 128-row tile within the portion, range). range < 0:
// the entry covers all key tiles of its query tile and its items write the attention output. Otherwise the entry is a
// piece of a query tile that has few rows and many keys, cut along the keys so that more SMs work on it: key tiles
// (range & 0xffff) .. + (range >> 16) - 1 of the tile's, and its items leave the unnormalised output and (maximum, sum)
// of their rows in the float32 scratch slot of the entry, which `attn_prefill_merge_kernel` merges in entry order.
__device__ __forceinline__ void entry_range(int range, int entry, int& k_begin, int& n_key_tiles, int& slot) {
  slot = -1;
  if (range < 0) return;
  const int lo = range & 0xffff, cnt = range >> 16;
  n_key_tiles = max(0, min(cnt, n_key_tiles - lo));
  k_begin += lo * BN;
  slot = entry;
}

// Item number `i` of this block. Items are numbered with the tiles in the host's order (most keys first) and the heads
// within a tile; the blocks take them in rows of gridDim.x items, every other row backwards, so that the block with the
// heaviest item of one row gets the lightest of the next.
__device__ __forceinline__ bool get_item(int i, int n_tiles, int Hq, const int* __restrict__ seg, const int* __restrict__ tiles,
                                         int window, Item& it) {
  const int G = gridDim.x, c = (i & 1) ? G - 1 - (int)blockIdx.x : (int)blockIdx.x;
  const long long k = (long long)i * G + c;
  if (k >= (long long)n_tiles * Hq) return false;
  const int ti = (int)(k / Hq);
  it.h = (int)(k - (long long)ti * Hq);
  it.s_idx = tiles[3 * ti];
  const int r_off = tiles[3 * ti + 1];
  it.n_key_tiles = 0;
  it.slot = -1;
  if (it.s_idx >= 0) {
    const int n_rows = seg[4 * it.s_idx + 1], pos0 = seg[4 * it.s_idx + 2];
    it.row = seg[4 * it.s_idx] + r_off;
    it.valid_rows = min(BM, n_rows - r_off);
    it.qpos0 = pos0 + r_off;
    it.last_pos = it.qpos0 + it.valid_rows - 1;
    it.lo_tile = window > 0 ? max(0, it.qpos0 - window + 1) : 0;
    it.k_begin = it.lo_tile & ~(BN - 1);
    it.n_key_tiles = (it.last_pos - it.k_begin) / BN + 1;
    entry_range(tiles[3 * ti + 2], ti, it.k_begin, it.n_key_tiles, it.slot);
  }
  return true;
}

// A row's share of an item's result that is a piece along the keys: this thread's `OD` dimensions of the unnormalised
// output from tensor memory (every lane of the warp takes part in the loads) and, from the thread of the row's first
// half, the maximum in use and the sum of weights.
template <int HD, int OD>
__device__ __forceinline__ void store_piece(uint32_t t_o, float* __restrict__ part_o, float* __restrict__ part_ml, size_t slot_row,
                                            int hf, bool valid, float m_run, float l_run) {
  float* dst = part_o + slot_row * HD + hf * OD;
#pragma unroll
  for (int c = 0; c < OD; c += 32) {
    float ov[32];
    tmem_ld32(t_o + (uint32_t)c, ov);
    if (valid) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) *(float4*)(dst + c + j) = make_float4(ov[j], ov[j + 1], ov[j + 2], ov[j + 3]);
    }
  }
  if (valid && hf == 0) *(float2*)(part_ml + slot_row * 2) = make_float2(m_run, l_run);
}

template <int HD, int BOX>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map,
                       const int* __restrict__ seg, const int* __restrict__ tiles, int n_tiles, const int* __restrict__ table,
                       int mb, int page_size, __nv_bfloat16* __restrict__ out, int Hq, int Hkv, float scale_log2, int window,
                       float* __restrict__ part_o, float* __restrict__ part_ml, int* err) {
  constexpr int HALVES = HD / 64;                     // 64-column halves of a head
  constexpr int KV_STAGES = HD <= 64 ? 4 : 3;         // key tiles and value tiles in flight (what shared memory holds)
  constexpr int HALF_BYTES = 128 * 128;               // 128 rows of 128 bytes
  constexpr int Q_BYTES = HALVES * HALF_BYTES, KV_BYTES = HALVES * HALF_BYTES;
  constexpr int TMEM_COLS = 512;                      // S: columns 0..127 and 128..255 (P over their first 64); O: 256..
  constexpr int OPS = (BN / BOX) * HALVES;            // TMA boxes per key tile, for K and again for V
  constexpr int OD = HD / 2;                          // output dimensions per thread
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  // [Q][K ring][V ring][row maxima][barriers]
  const uint32_t s_q = smem_u32(smem), s_k = s_q + Q_BYTES, s_v = s_k + KV_STAGES * KV_BYTES;
  float* s_mx = (float*)(smem + Q_BYTES + 2 * KV_STAGES * KV_BYTES);      // [2 halves][128 rows]
  uint64_t* bars = (uint64_t*)(s_mx + 2 * BM);
  uint64_t* q_full = bars;                 // 1
  uint64_t* q_empty = bars + 1;            // 1
  uint64_t* k_full = bars + 2;             // KV_STAGES each
  uint64_t* k_empty = k_full + KV_STAGES;
  uint64_t* v_full = k_empty + KV_STAGES;
  uint64_t* v_empty = v_full + KV_STAGES;
  uint64_t* s_ready = v_empty + KV_STAGES; // 2: one per S buffer
  uint64_t* p_ready = s_ready + 2;         // 2: one per P buffer
  uint64_t* pv_ready = p_ready + 2;        // 2: PV of the even and of the odd key tiles
  uint32_t* tmem_slot = (uint32_t*)(pv_ready + 2);
  int* flag = (int*)(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_ready[i], 1);
      mbar_init(&p_ready[i], 256);
      mbar_init(&pv_ready[i], 1);
    }
    flag[0] = 0;
    mbar_init_fence();
  }
  // zeros in the key / value stages: a box that is not fetched (keys past the portion's last position) must not hold
  // another kernel's bits, since P = 0 times NaN is NaN (what an earlier item of this block left there is finite)
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
  fz_grid_wait();
  // Every role walks the same items in the same order and counts the key tiles it has gone through (`g`): ring stages,
  // buffers and barrier phases follow from that count, so they carry over from one item to the next, and the producers
  // fetch the next item's tiles while the softmax warps still work on this one's.

  if (warp == 0 || warp == 10) {
    // ---------------- TMA producers: warp 0 the Q tile and the key tiles, warp 10 the value tiles; each runs as far
    // ahead as its ring allows (a key stage is free once its score product is done, a value stage once its PV is)
    const bool is_v = warp == 10;
    const int rows_per_page = 2 * Hkv * page_size;
    bool ok = true;
    int g = 0, n_q = 0;
    Item it;
    for (int i = 0; ok && get_item(i, n_tiles, Hq, seg, tiles, window, it); ++i) {
      if (it.n_key_tiles == 0) continue;
      const int kvh = it.h / (Hq / Hkv);
      if (!is_v) {
        // the one Q buffer is free once the last score product of the item before is done
        if (n_q > 0) ok = __all_sync(0xffffffffu, mbar_wait(q_empty, (n_q - 1) & 1));
        if (!ok) break;
        if (lane == 0) {
          mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
          for (int hf = 0; hf < HALVES; ++hf) tma_load_2d_u32(s_q + hf * HALF_BYTES, &q_map, smem_u32(q_full), it.h * HD + 64 * hf, it.row);
        }
        ++n_q;
      }
      const int* trow = table + (size_t)it.s_idx * mb;
      for (int t = 0; t < it.n_key_tiles && ok; ++t, ++g) {
        const int s = g % KV_STAGES, round = g / KV_STAGES;
        const int key0 = it.k_begin + t * BN;
        // op -> (page box, column half); a box is fetched if any of its keys lies in [lo_tile, last_pos]
        int op_row[(OPS + 31) / 32];
        uint32_t bytes = 0;
#pragma unroll
        for (int j = 0; j < (OPS + 31) / 32; ++j) {
          const int op = lane + 32 * j;
          op_row[j] = -1;
          if (op < OPS) {
            const int box = op / HALVES;
            const int key = key0 + box * BOX;
            if (key <= it.last_pos && key + BOX - 1 >= it.lo_tile) {
              const int pi = key / page_size;
              const int page = trow[pi];
              if (page >= 0) op_row[j] = page * rows_per_page + kvh * page_size + (key - pi * page_size);
              else if (!is_v) atomicOr(err, FZ_ERR_NO_PAGE);
            }
          }
          bytes += op_row[j] >= 0 ? BOX * 128u : 0u;
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
        for (int j = 0; j < (OPS + 31) / 32; ++j) {
          const int op = lane + 32 * j;
          if (op < OPS && op_row[j] >= 0) {
            const int box = op / HALVES, hf = op % HALVES;
            tma_load_2d_u32(dst + hf * HALF_BYTES + box * BOX * 128, &kv_map, bar, 64 * hf, op_row[j] + (is_v ? Hkv * page_size : 0));
          }
        }
      }
    }
    if (!ok && lane == 0) flag[0] = 1;
  } else if (warp == 1) {
    // ---------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(BM, BN, false), idesc_pv = make_idesc(BM, HD, true);
      bool ok = true;
      int g0 = 0, n_q = 0;
      auto issue_s = [&](int g) -> bool {      // S(g) = Q K(g)^T into S buffer g & 1; frees the key stage when done
        const int s = g % KV_STAGES;
        if (!mbar_wait(&k_full[s], (g / KV_STAGES) & 1)) return false;
        tc_fence_after();
        const uint32_t sk = s_k + s * KV_BYTES, tmem_s = tmem_base + (uint32_t)(g & 1) * 128u;
#pragma unroll
        for (int hf = 0; hf < HALVES; ++hf) {
          const uint64_t dq = desc_k_major(s_q + hf * HALF_BYTES), dk = desc_k_major(sk + hf * HALF_BYTES);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_bf16(tmem_s, dq + (uint64_t)(2 * k), dk + (uint64_t)(2 * k), idesc_s, (hf | k) ? 1u : 0u);
        }
        umma_commit(&s_ready[g & 1]);
        umma_commit(&k_empty[s]);
        return true;
      };
      Item it;
      for (int i = 0; ok && get_item(i, n_tiles, Hq, seg, tiles, window, it); ++i) {
        if (it.n_key_tiles == 0) continue;
        const int T = it.n_key_tiles;
        ok = mbar_wait(q_full, n_q & 1);
        ++n_q;
        if (ok) ok = issue_s(g0);
        if (ok && T == 1) umma_commit(q_empty);
        for (int t = 0; t < T && ok; ++t) {
          const int g = g0 + t;
          // the next tile's scores run on the tensor core while the softmax warps work on this tile's
          if (t + 1 < T) {
            if (!issue_s(g + 1)) { ok = false; break; }
            if (t + 2 == T) umma_commit(q_empty);       // the item's last score product: Q may be overwritten when it is done
          }
          const int s = g % KV_STAGES, b = g & 1;
          if (!mbar_wait(&v_full[s], (g / KV_STAGES) & 1)) { ok = false; break; }
          if (!mbar_wait(&p_ready[b], (g >> 1) & 1)) { ok = false; break; }       // P(g) written, O rescaled if it had to be
          tc_fence_after();
          const uint32_t sv = s_v + s * KV_BYTES, tmem_p = tmem_base + (uint32_t)b * 128u, tmem_o = tmem_base + 256u;
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk) {
            const uint64_t dv = desc_mn_major(sv + kk * 16 * 128, HALF_BYTES);
            umma_bf16_a_tmem(tmem_o, tmem_p + (uint32_t)(8 * kk), dv, idesc_pv, (t | kk) ? 1u : 0u);
          }
          umma_commit(&pv_ready[b]);
          umma_commit(&v_empty[s]);
        }
        g0 += T;
      }
      if (!ok) flag[0] = 1;
    }
  } else {
    // ---------------- softmax and output: two threads per row
    const int quad = warp & 3, hf = (warp - 2) >> 2;          // warps w and w + 4 share the row quarter `quad`
    const int r = quad * 32 + lane;
    const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
    const int pair_bar = 1 + quad;                             // named barrier of the two warps of this row quarter
    const uint32_t t_o = tmem_base + 256u + (uint32_t)(hf * OD) + lane_sel;      // this thread's half of the output dimensions
    bool ok = true;
    int g0 = 0;
    Item it;
    for (int i = 0; ok && get_item(i, n_tiles, Hq, seg, tiles, window, it); ++i) {
      if (it.n_key_tiles == 0) {
        // (a piece that a layer's window leaves without keys: its rows weigh nothing in the merge)
        if (it.slot >= 0 && hf == 0 && r < it.valid_rows)
          *(float2*)(part_ml + (((size_t)it.slot * Hq + it.h) * BM + r) * 2) = make_float2(-INFINITY, 0.f);
        continue;
      }
      const int T = it.n_key_tiles, qpos = it.qpos0 + r;
      float m_run = -INFINITY, l_part = 0.f;      // the maximum in use (exp2 domain) and this thread's half of the row's sum
      for (int t = 0; t < T && ok; ++t) {
        const int g = g0 + t, b = g & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(&s_ready[b], (g >> 1) & 1));
        if (!ok) break;
        tc_fence_after();
        const uint32_t t_s = tmem_base + (uint32_t)b * 128u + (uint32_t)(hf * 64) + lane_sel;
        const int key0 = it.k_begin + t * BN + hf * 64;
        const int lo_key = window > 0 ? max(it.lo_tile, qpos - window + 1) : it.lo_tile;
        const bool full = key0 + 63 <= qpos && key0 >= lo_key;     // every key of this thread's half is visible to its row
        float v[64];
        tmem_ld32(t_s, v);
        tmem_ld32(t_s + 32u, v + 32);
        if (!full) {
#pragma unroll
          for (int j = 0; j < 64; ++j) {
            const int key = key0 + j;
            v[j] = (key <= qpos && key >= lo_key) ? v[j] : -INFINITY;      // exp2(-inf) = 0 below
          }
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};       // four chains, so that the maxima do not wait on one another
#pragma unroll
        for (int j = 0; j < 64; j += 8) {
          mx4[0] = fmax3(mx4[0], v[j], v[j + 1]); mx4[1] = fmax3(mx4[1], v[j + 2], v[j + 3]);
          mx4[2] = fmax3(mx4[2], v[j + 4], v[j + 5]); mx4[3] = fmax3(mx4[3], v[j + 6], v[j + 7]);
        }
        float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        // the row's maximum over both halves
        s_mx[hf * BM + r] = mx;
        asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
        mx = fmaxf(mx, s_mx[(hf ^ 1) * BM + r]);
        asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");    // both have read: the slots may be written again
        // The output accumulates in tensor memory over the item's key tiles and is rescaled there only when the row's
        // maximum has grown by more than 2^RESCALE_STEP over the maximum in use (P then stays below 2^RESCALE_STEP:
        // harmless in bf16 and in the float32 sums; the maximum in use cancels in the final division). That is rare
        // after the first tiles, and the output does not take up registers meanwhile.
        const float m_new = fmaxf(m_run, mx * scale_log2);
        const bool grow = m_new > m_run + RESCALE_STEP;          // (-inf + step = -inf: the first finite maximum counts)
        if (__any_sync(0xffffffffu, grow)) {
          const float corr = grow ? fast_exp2(m_run - m_new) : 1.f;
          if (t > 0) {
            ok = __all_sync(0xffffffffu, mbar_wait(&pv_ready[(g - 1) & 1], ((g - 1) >> 1) & 1));      // PV(g - 1) is in
            if (!ok) break;
            tc_fence_after();
            const float2 c2 = make_float2(corr, corr);
#pragma unroll
            for (int c = 0; c < OD; c += 32) {
              float ov[32];
              tmem_ld32(t_o + (uint32_t)c, ov);
              uint32_t ow[32];
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float2 sc = __fmul2_rn(make_float2(ov[2 * j], ov[2 * j + 1]), c2);
                ow[2 * j] = __float_as_uint(sc.x);
                ow[2 * j + 1] = __float_as_uint(sc.y);
              }
              tmem_st32(t_o + (uint32_t)c, ow);
            }
          }
          if (grow) {
            l_part *= corr;
            m_run = m_new;
          }
        }
        const float mu = m_run == -INFINITY ? 0.f : m_run;
        // P goes back into tensor memory as the A operand of the PV product: bf16 pairs, over the first 64 columns of
        // the score buffer (both threads of the row have read their scores: the pair barrier above lies between).
        // Where every key of this thread's half is visible (no -inf), three pairs of exponentials in eight run on the
        // FMA pipe: that balances it with the special-function unit.
        const float2 sc2 = make_float2(scale_log2, scale_log2), nmu2 = make_float2(-mu, -mu);
        float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};      // two packed chains; added up in a fixed order below
        uint32_t w[32];
        if (full) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float2 x = __ffma2_rn(make_float2(v[2 * j], v[2 * j + 1]), sc2, nmu2);
            const float2 e = ((0x52u >> (j & 7)) & 1u) ? exp2_fma2(x) : make_float2(fast_exp2(x.x), fast_exp2(x.y));      // 3 pairs in 8
            sum2[j & 1] = __fadd2_rn(sum2[j & 1], e);
            const __nv_bfloat162 pk = __floats2bfloat162_rn(e.x, e.y);
            w[j] = *(const uint32_t*)&pk;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float2 x = __ffma2_rn(make_float2(v[2 * j], v[2 * j + 1]), sc2, nmu2);
            const float2 e = make_float2(fast_exp2(x.x), fast_exp2(x.y));
            sum2[j & 1] = __fadd2_rn(sum2[j & 1], e);
            const __nv_bfloat162 pk = __floats2bfloat162_rn(e.x, e.y);
            w[j] = *(const uint32_t*)&pk;
          }
        }
        l_part += (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);
        __syncwarp();      // (the store to tensor memory is a warp-wide instruction; `full` differs between lanes)
        tmem_st32(tmem_base + (uint32_t)b * 128u + (uint32_t)(hf * 32) + lane_sel, w);
        tc_fence_before();
        mbar_arrive(&p_ready[b]);
      }
      if (!ok) break;
      g0 += T;
      ok = __all_sync(0xffffffffu, mbar_wait(&pv_ready[(g0 - 1) & 1], ((g0 - 1) >> 1) & 1));      // the item's last PV
      if (!ok) break;
      tc_fence_after();
      // the row's sum of weights: half 0 + half 1
      s_mx[hf * BM + r] = l_part;
      asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
      const float l_run = s_mx[r] + s_mx[BM + r];
      asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");    // both have read: the slots may be written again
      if (it.slot >= 0) {      // a piece along the keys: the merge kernel finishes the rows
        store_piece<HD, OD>(t_o, part_o, part_ml, ((size_t)it.slot * Hq + it.h) * BM + r, hf, r < it.valid_rows, m_run, l_run);
        tc_fence_before();
        continue;
      }
      const float inv = 1.0f / l_run;
      __nv_bfloat16* orow = out + (size_t)(it.row + r) * Hq * HD + (size_t)it.h * HD + hf * OD;
      // (the loads from tensor memory are warp-wide instructions: every lane takes part, rows past the portion's end
      // just do not store. The next item's first PV overwrites O only after every thread has arrived with its first P,
      // which it does after these loads.)
#pragma unroll
      for (int c = 0; c < OD; c += 32) {
        float ov[32];
        tmem_ld32(t_o + (uint32_t)c, ov);
        if (r < it.valid_rows) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint32_t w[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const __nv_bfloat162 pk = __floats2bfloat162_rn(ov[j + 2 * q] * inv, ov[j + 2 * q + 1] * inv);
              w[q] = *(const uint32_t*)&pk;
            }
            *(uint4*)(orow + c + j) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      tc_fence_before();
    }
    if (!ok) flag[0] = 1;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (tid == 0 && flag[0]) atomicOr(err, FZ_ERR_WAIT_TIMEOUT);
}

// ------------------------------------------------------------------------------------------------ two heads per block
// The same attention with TWO query tiles per block: the same 128 token rows for two query heads of one kv head. Both
// tiles read the same key and value stages (each stage is fetched once and used twice), and each tile has its own score
// / probability columns and its own output columns in tensor memory and its own eight softmax warps (two threads per
// row, each with 64 of the tile's 128 score columns and half of the output dimensions; one warp alone on a scheduler
// leaves most of its issue slots empty, two keep it busy). A thread writes its P over the first half of its own scores,
// so nobody overwrites what the other thread of the row still reads. The one MMA lane alternates between the
// tiles: S0 = Q0 K^T, S1 = Q1 K^T, then as each tile's P arrives O0 += P0 V, S0' = Q0 K'^T, O1 += P1 V, S1' = Q1 K'^T ...
// so one tile's exponentials run while the tensor core works for the other tile, instead of the tensor core idling
// through every tile's softmax. Within a tile the chain S -> softmax -> P V -> next S is serial (P lies over the scores
// it came from, so the next scores of a tile are issued behind its P V product; MMAs of one thread run in issue order).
// A kv head with an odd number of query heads has one item with a single tile (`active1 == 0`).
#ifdef FZ_ATTN_PROF
__device__ unsigned long long fz_attn_prof[32];
#define PROF_T(x) const long long x = clock64()
#define PROF_ADD(i, v) do { if (prof_on) atomicAdd(&fz_attn_prof[i], (unsigned long long)(v)); } while (0)
#else
#define PROF_T(x)
#define PROF_ADD(i, v)
#endif
struct PairItem {
  int n_key_tiles, s_idx, h0, active1, kvh, row, valid_rows, qpos0, last_pos, lo_tile, k_begin, slot;
};

__device__ __forceinline__ bool get_pair_item(int i, int n_tiles, int Hq, int Hkv, const int* __restrict__ seg,
                                              const int* __restrict__ tiles, int window, PairItem& it) {
  const int G = gridDim.x, c = (i & 1) ? G - 1 - (int)blockIdx.x : (int)blockIdx.x;
  const int gq = Hq / Hkv, ppg = (gq + 1) >> 1, pairs = Hkv * ppg;
  const long long k = (long long)i * G + c;
  if (k >= (long long)n_tiles * pairs) return false;
  const int ti = (int)(k / pairs), pr = (int)(k - (long long)ti * pairs);
  it.kvh = pr / ppg;
  const int j = pr - it.kvh * ppg;
  it.h0 = it.kvh * gq + 2 * j;
  it.active1 = 2 * j + 1 < gq;
  it.s_idx = tiles[3 * ti];
  const int r_off = tiles[3 * ti + 1];
  it.n_key_tiles = 0;
  it.slot = -1;
  if (it.s_idx >= 0) {
    const int n_rows = seg[4 * it.s_idx + 1], pos0 = seg[4 * it.s_idx + 2];
    it.row = seg[4 * it.s_idx] + r_off;
    it.valid_rows = min(BM, n_rows - r_off);
    it.qpos0 = pos0 + r_off;
    it.last_pos = it.qpos0 + it.valid_rows - 1;
    it.lo_tile = window > 0 ? max(0, it.qpos0 - window + 1) : 0;
    it.k_begin = it.lo_tile & ~(BN - 1);
    it.n_key_tiles = (it.last_pos - it.k_begin) / BN + 1;
    entry_range(tiles[3 * ti + 2], ti, it.k_begin, it.n_key_tiles, it.slot);
  }
  return true;
}

template <int HD, int BOX>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
attn_prefill_pair_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map,
                         const int* __restrict__ seg, const int* __restrict__ tiles, int n_tiles, const int* __restrict__ table,
                         int mb, int page_size, __nv_bfloat16* __restrict__ out, int Hq, int Hkv, float scale_log2, int window,
                         float* __restrict__ part_o, float* __restrict__ part_ml, int* err) {
  constexpr int HALVES = HD / 64;
  constexpr int KV_STAGES = HD <= 64 ? 4 : 2;         // key tiles and value tiles in flight
  constexpr int HALF_BYTES = 128 * 128;
  constexpr int Q_BYTES = HALVES * HALF_BYTES, KV_BYTES = HALVES * HALF_BYTES;
  constexpr int TMEM_COLS = 512;                      // S0 / P0: 0.., S1 / P1: 128.., O0: 256.., O1: 256 + HD..
  constexpr int OPS = (BN / BOX) * HALVES;
  constexpr int OD = HD / 2;                          // output dimensions per thread
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  // [Q0][Q1][K ring][V ring][row maxima / sums][barriers]
  const uint32_t s_q = smem_u32(smem), s_k = s_q + 2 * Q_BYTES, s_v = s_k + KV_STAGES * KV_BYTES;
  float* s_mx = (float*)(smem + 2 * Q_BYTES + 2 * KV_STAGES * KV_BYTES);      // [2 tiles][2 halves][128 rows]
  uint64_t* bars = (uint64_t*)(s_mx + 4 * BM);
  uint64_t* q_full = bars;
  uint64_t* q_empty = bars + 1;
  uint64_t* k_full = bars + 2;
  uint64_t* k_empty = k_full + KV_STAGES;
  uint64_t* v_full = k_empty + KV_STAGES;
  uint64_t* v_empty = v_full + KV_STAGES;
  uint64_t* s_ready = v_empty + KV_STAGES;  // [2]: the scores of tile 0 / 1 are in
  uint64_t* p_ready = s_ready + 2;          // [2]: 128 arrivals each: P of the tile is written (O rescaled if it had to be)
  uint64_t* o_ready = p_ready + 2;          // [2]: the item's last P V product of the tile is done
  uint32_t* tmem_slot = (uint32_t*)(o_ready + 2);
  int* flag = (int*)(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_ready[i], 1);
      mbar_init(&p_ready[i], 256);
      mbar_init(&o_ready[i], 1);
    }
    flag[0] = 0;
    mbar_init_fence();
  }
  // zeros in the key / value stages (see the kernel above)
  for (int e = tid; e < 2 * KV_STAGES * KV_BYTES / 16; e += PAIR_THREADS) ((uint4*)(smem + 2 * Q_BYTES))[e] = make_uint4(0u, 0u, 0u, 0u);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  fz_grid_launch_dependents();
  fz_grid_wait();

  if (warp == 0 || warp == 18) {
    // ---------------- TMA producers: warp 0 the two Q tiles and the key tiles, warp 18 the value tiles
    const bool is_v = warp == 18;
    const int rows_per_page = 2 * Hkv * page_size;
    bool ok = true;
    int g = 0, n_q = 0;
    PairItem it;
    for (int i = 0; ok && get_pair_item(i, n_tiles, Hq, Hkv, seg, tiles, window, it); ++i) {
      if (it.n_key_tiles == 0) continue;
      if (!is_v) {
        if (n_q > 0) ok = __all_sync(0xffffffffu, mbar_wait(q_empty, (n_q - 1) & 1));
        if (!ok) break;
        if (lane == 0) {
          mbar_expect_tx(q_full, (1 + it.active1) * Q_BYTES);
          for (int tq = 0; tq <= it.active1; ++tq)
#pragma unroll
            for (int hf = 0; hf < HALVES; ++hf)
              tma_load_2d_u32(s_q + tq * Q_BYTES + hf * HALF_BYTES, &q_map, smem_u32(q_full), (it.h0 + tq) * HD + 64 * hf, it.row);
        }
        ++n_q;
      }
      const int* trow = table + (size_t)it.s_idx * mb;
      for (int t = 0; t < it.n_key_tiles && ok; ++t, ++g) {
        const int s = g % KV_STAGES, round = g / KV_STAGES;
        const int key0 = it.k_begin + t * BN;
        int op_row[(OPS + 31) / 32];
        uint32_t bytes = 0;
#pragma unroll
        for (int j = 0; j < (OPS + 31) / 32; ++j) {
          const int op = lane + 32 * j;
          op_row[j] = -1;
          if (op < OPS) {
            const int box = op / HALVES;
            const int key = key0 + box * BOX;
            if (key <= it.last_pos && key + BOX - 1 >= it.lo_tile) {
              const int pi = key / page_size;
              const int page = trow[pi];
              if (page >= 0) op_row[j] = page * rows_per_page + it.kvh * page_size + (key - pi * page_size);
              else if (!is_v) atomicOr(err, FZ_ERR_NO_PAGE);
            }
          }
          bytes += op_row[j] >= 0 ? BOX * 128u : 0u;
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
        for (int j = 0; j < (OPS + 31) / 32; ++j) {
          const int op = lane + 32 * j;
          if (op < OPS && op_row[j] >= 0) {
            const int box = op / HALVES, hf = op % HALVES;
            tma_load_2d_u32(dst + hf * HALF_BYTES + box * BOX * 128, &kv_map, bar, 64 * hf, op_row[j] + (is_v ? Hkv * page_size : 0));
          }
        }
      }
    }
    if (!ok && lane == 0) flag[0] = 1;
  } else if (warp == 1) {
    // ---------------- MMA issuer: one lane for both tiles. (One lane per tile was tried: the two interleave their
    // instructions on the tensor core and the whole is slower.)
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(BM, BN, false), idesc_pv = make_idesc(BM, HD, true);
      bool ok = true;
      int g0 = 0, n_q = 0;
      int n_p[2] = {0, 0};          // key tiles whose P has been consumed, per Q tile (the phase of p_ready)
#ifdef FZ_ATTN_PROF
      const bool prof_on = blockIdx.x == 3;
      const long long m_begin = clock64();
#endif
      auto issue_s = [&](int tq, int g) {      // S_tq(g) = Q_tq K(g)^T; the caller has waited for the key stage
        PROF_T(s0);
        const uint32_t sk = s_k + (g % KV_STAGES) * KV_BYTES, sq = s_q + tq * Q_BYTES, tmem_s = tmem_base + (uint32_t)tq * 128u;
#pragma unroll
        for (int hf = 0; hf < HALVES; ++hf) {
          const uint64_t dq = desc_k_major(sq + hf * HALF_BYTES), dk = desc_k_major(sk + hf * HALF_BYTES);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_bf16(tmem_s, dq + (uint64_t)(2 * k), dk + (uint64_t)(2 * k), idesc_s, (hf | k) ? 1u : 0u);
        }
        umma_commit(&s_ready[tq]);
        PROF_T(s1);
        PROF_ADD(22, s1 - s0);
      };
      auto issue_pv = [&](int tq, int g, bool first) -> bool {      // O_tq (+)= P_tq(g) V(g), once the tile's P is in
        PROF_T(w0);
        if (!mbar_wait(&p_ready[tq], n_p[tq] & 1)) return false;
        PROF_T(w1);
        PROF_ADD(16 + tq, w1 - w0);
        ++n_p[tq];
        tc_fence_after();
        const uint32_t sv = s_v + (g % KV_STAGES) * KV_BYTES, tmem_p = tmem_base + (uint32_t)tq * 128u;
        const uint32_t tmem_o = tmem_base + 256u + (uint32_t)(tq * HD);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const uint64_t dv = desc_mn_major(sv + kk * 16 * 128, HALF_BYTES);
          // (keys 0..63 of the tile: P words at columns 0..31; keys 64..127: at columns 64..95)
          umma_bf16_a_tmem(tmem_o, tmem_p + (uint32_t)(kk < 4 ? 8 * kk : 32 + 8 * kk), dv, idesc_pv, (!first || kk) ? 1u : 0u);
        }
        PROF_T(w2);
        PROF_ADD(23, w2 - w1);
        return true;
      };
      PairItem it;
      for (int i = 0; ok && get_pair_item(i, n_tiles, Hq, Hkv, seg, tiles, window, it); ++i) {
        if (it.n_key_tiles == 0) continue;
        const int T = it.n_key_tiles, last_tq = it.active1;
        ok = mbar_wait(q_full, n_q & 1);
        ++n_q;
        if (ok) ok = mbar_wait(&k_full[g0 % KV_STAGES], (g0 / KV_STAGES) & 1);
        if (!ok) break;
        tc_fence_after();
        for (int tq = 0; tq <= last_tq; ++tq) issue_s(tq, g0);
        umma_commit(&k_empty[g0 % KV_STAGES]);
        if (T == 1) umma_commit(q_empty);
        for (int t = 0; t < T && ok; ++t) {
          const int g = g0 + t;
          const bool more = t + 1 < T;
          PROF_T(v0);
          if (!mbar_wait(&v_full[g % KV_STAGES], (g / KV_STAGES) & 1)) { ok = false; break; }
          PROF_T(v1);
          PROF_ADD(18, v1 - v0);
          for (int tq = 0; tq <= last_tq && ok; ++tq) {
            if (!issue_pv(tq, g, t == 0)) { ok = false; break; }
            if (!more) umma_commit(&o_ready[tq]);
            if (tq == last_tq) umma_commit(&v_empty[g % KV_STAGES]);
            if (more) {
              // the tile's next scores go behind its P V product (they overwrite the P it reads)
              PROF_T(k0);
              if (tq == 0 && !mbar_wait(&k_full[(g + 1) % KV_STAGES], ((g + 1) / KV_STAGES) & 1)) { ok = false; break; }
              PROF_T(k1);
              PROF_ADD(19, k1 - k0);
              if (tq == 0) tc_fence_after();
              issue_s(tq, g + 1);
              if (tq == last_tq) {
                umma_commit(&k_empty[(g + 1) % KV_STAGES]);
                if (t + 2 == T) umma_commit(q_empty);      // the item's last score products: Q may be overwritten when they are done
              }
            }
          }
        }
        g0 += T;
      }
#ifdef FZ_ATTN_PROF
      PROF_ADD(20, clock64() - m_begin);
      PROF_ADD(21, g0);
#endif
      if (!ok) flag[0] = 1;
    }
  } else {
    // ---------------- softmax and output: warps 2..9 tile 0, warps 10..17 tile 1; two threads per row
    const int idx = warp - 2, tq = idx >> 3, hf = (idx >> 2) & 1, quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
    const uint32_t t_s = tmem_base + (uint32_t)(tq * 128 + hf * 64) + lane_sel;    // this thread's 64 scores; its P over the first 32 columns
    const uint32_t t_o = tmem_base + 256u + (uint32_t)(tq * HD + hf * OD) + lane_sel;
    const int pair_bar = 1 + tq * 4 + quad;                    // named barrier of the two warps that share these rows
    float* mx_mine = s_mx + (tq * 2 + hf) * BM + r;
    const float* mx_other = s_mx + (tq * 2 + (hf ^ 1)) * BM + r;
    bool ok = true;
    int n_s = 0, n_items = 0;      // key tiles and items this tile has gone through (the phases of s_ready and o_ready)
    PairItem it;
    for (int i = 0; ok && get_pair_item(i, n_tiles, Hq, Hkv, seg, tiles, window, it); ++i) {
      if (tq > it.active1) continue;
      if (it.n_key_tiles == 0) {
        // (a piece that a layer's window leaves without keys: its rows weigh nothing in the merge)
        if (it.slot >= 0 && hf == 0 && r < it.valid_rows)
          *(float2*)(part_ml + (((size_t)it.slot * Hq + (it.h0 + tq)) * BM + r) * 2) = make_float2(-INFINITY, 0.f);
        continue;
      }
      const int T = it.n_key_tiles, qpos = it.qpos0 + r;
      const int lo_key = window > 0 ? max(it.lo_tile, qpos - window + 1) : it.lo_tile;
      float m_run = -INFINITY, l_part = 0.f;      // the maximum in use and this thread's half of the row's sum
      for (int t = 0; t < T && ok; ++t) {
#ifdef FZ_ATTN_PROF
        const bool prof_on = blockIdx.x == 3 && lane == 0 && quad == 0 && hf == 0;
#endif
        PROF_T(c0);
        ok = __all_sync(0xffffffffu, mbar_wait(&s_ready[tq], n_s & 1));
        if (!ok) break;
        ++n_s;
        tc_fence_after();
        PROF_T(c1);
        const int key0 = it.k_begin + t * BN + hf * 64;
        const bool full = key0 + 63 <= qpos && key0 >= lo_key;      // every key of this thread's half is visible to its row
        // pass 1: the maximum of this thread's 64 scores, then of the row
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < 64; c += 32) {
          float v[32];
          tmem_ld32(t_s + (uint32_t)c, v);
          if (!full) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int key = key0 + c + j;
              v[j] = (key <= qpos && key >= lo_key) ? v[j] : -INFINITY;
            }
          }
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            mx4[0] = fmax3(mx4[0], v[j], v[j + 1]); mx4[1] = fmax3(mx4[1], v[j + 2], v[j + 3]);
            mx4[2] = fmax3(mx4[2], v[j + 4], v[j + 5]); mx4[3] = fmax3(mx4[3], v[j + 6], v[j + 7]);
          }
        }
        float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        PROF_T(c2);
        *mx_mine = mx;
        asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
        mx = fmaxf(mx, *mx_other);
        asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");    // both have read: the slots may be written again
        PROF_T(c3);
        // O stays in tensor memory and is rescaled there only when the row's maximum has grown by more than
        // 2^RESCALE_STEP over the maximum in use. The tile's last P V product is complete by now: the scores just waited
        // for were issued behind it, and their completion is signalled after that of everything issued before.
        const float m_new = fmaxf(m_run, mx * scale_log2);
        const bool grow = m_new > m_run + RESCALE_STEP;
        if (__any_sync(0xffffffffu, grow)) {
          const float corr = grow ? fast_exp2(m_run - m_new) : 1.f;
          if (t > 0) {
            const float2 c2 = make_float2(corr, corr);
#pragma unroll
            for (int c = 0; c < OD; c += 32) {
              float ov[32];
              tmem_ld32(t_o + (uint32_t)c, ov);
              uint32_t ow[32];
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float2 sc = __fmul2_rn(make_float2(ov[2 * j], ov[2 * j + 1]), c2);
                ow[2 * j] = __float_as_uint(sc.x);
                ow[2 * j + 1] = __float_as_uint(sc.y);
              }
              tmem_st32(t_o + (uint32_t)c, ow);
            }
          }
          if (grow) {
            l_part *= corr;
            m_run = m_new;
          }
        }
        const float mu = m_run == -INFINITY ? 0.f : m_run;
        PROF_T(c4);
        // pass 2: P = exp2(s * scale - mu) as bf16 pairs, 32 scores at a time; the 16 words of a chunk go over the first
        // half of this thread's own scores (words 0..15 over scores 0..15, words 16..31 over scores 16..31: read before).
        // Where every key is visible, three pairs of exponentials in eight run on the FMA pipe.
        const float2 sc2 = make_float2(scale_log2, scale_log2), nmu2 = make_float2(-mu, -mu);
        float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
        for (int c = 0; c < 64; c += 32) {
          float v[32];
          tmem_ld32(t_s + (uint32_t)c, v);
          uint32_t w[16];
          if (full) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float2 x = __ffma2_rn(make_float2(v[2 * j], v[2 * j + 1]), sc2, nmu2);
              const float2 e = ((0x52u >> (j & 7)) & 1u) ? exp2_fma2(x) : make_float2(fast_exp2(x.x), fast_exp2(x.y));
              sum2[j & 1] = __fadd2_rn(sum2[j & 1], e);
              const __nv_bfloat162 pk = __floats2bfloat162_rn(e.x, e.y);
              w[j] = *(const uint32_t*)&pk;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int key = key0 + c + 2 * j;
              const float s0 = (key <= qpos && key >= lo_key) ? v[2 * j] : -INFINITY;
              const float s1 = (key + 1 <= qpos && key + 1 >= lo_key) ? v[2 * j + 1] : -INFINITY;
              const float2 x = __ffma2_rn(make_float2(s0, s1), sc2, nmu2);
              const float2 e = make_float2(fast_exp2(x.x), fast_exp2(x.y));
              sum2[j & 1] = __fadd2_rn(sum2[j & 1], e);
              const __nv_bfloat162 pk = __floats2bfloat162_rn(e.x, e.y);
              w[j] = *(const uint32_t*)&pk;
            }
          }
          __syncwarp();      // (the store to tensor memory is a warp-wide instruction; `full` differs between lanes)
          tmem_st16(t_s + (uint32_t)(c >> 1), w);
        }
        l_part += (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);
        PROF_T(c5);
        tc_fence_before();
        mbar_arrive(&p_ready[tq]);
        PROF_T(c6);
        PROF_ADD(tq * 8 + 0, c1 - c0); PROF_ADD(tq * 8 + 1, c2 - c1); PROF_ADD(tq * 8 + 2, c3 - c2); PROF_ADD(tq * 8 + 3, c4 - c3);
        PROF_ADD(tq * 8 + 4, c5 - c4); PROF_ADD(tq * 8 + 5, c6 - c5); PROF_ADD(tq * 8 + 6, 1);
      }
      if (!ok) break;
      ok = __all_sync(0xffffffffu, mbar_wait(&o_ready[tq], n_items & 1));      // the item's last P V product of this tile
      if (!ok) break;
      ++n_items;
      tc_fence_after();
      // the row's sum of weights: half 0 + half 1
      *mx_mine = l_part;
      asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
      const float l_run = s_mx[(tq * 2) * BM + r] + s_mx[(tq * 2 + 1) * BM + r];
      asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");    // both have read: the slots may be written again
      if (it.slot >= 0) {      // a piece along the keys: the merge kernel finishes the rows
        store_piece<HD, OD>(t_o, part_o, part_ml, ((size_t)it.slot * Hq + (it.h0 + tq)) * BM + r, hf, r < it.valid_rows, m_run, l_run);
        tc_fence_before();
        continue;
      }
      const float inv = 1.0f / l_run;
      __nv_bfloat16* orow = out + (size_t)(it.row + r) * Hq * HD + (size_t)(it.h0 + tq) * HD + hf * OD;
      // (loads from tensor memory are warp-wide: every lane takes part, rows past the portion's end just do not store)
#pragma unroll
      for (int c = 0; c < OD; c += 32) {
        float ov[32];
        tmem_ld32(t_o + (uint32_t)c, ov);
        if (r < it.valid_rows) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint32_t w[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const __nv_bfloat162 pk = __floats2bfloat162_rn(ov[j + 2 * q] * inv, ov[j + 2 * q + 1] * inv);
              w[q] = *(const uint32_t*)&pk;
            }
            *(uint4*)(orow + c + j) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      tc_fence_before();
    }
    if (!ok) flag[0] = 1;
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
int launch_pair(const void* q, int N, const void* k_pool, long long pool_rows, const int* seg, const int* tiles, int n_tiles,
                const int* table, int mb, int page_size, void* out, int Hq, int Hkv, float scale, int window, float* part_o,
                float* part_ml, int* err, cudaStream_t stream) {
  CUtensorMap qm, kvm;
  int st = get_map_bf16(q, N, Hq * HD, BM, &qm);
  if (st != FZ_OK) return st;
  if ((st = get_map_bf16(k_pool, pool_rows, HD, BOX, &kvm)) != FZ_OK) return st;
  constexpr int HALVES = HD / 64, HALF_BYTES = 128 * 128;
  constexpr int KV_STAGES = HD <= 64 ? 4 : 2;
  constexpr size_t smem = (size_t)2 * HALVES * HALF_BYTES + KV_STAGES * 2 * HALVES * HALF_BYTES + 4 * BM * 4 + 8 * 32 + 1024;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  static bool raised = false;
  if (!raised) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_pair_kernel<HD, BOX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    raised = true;
  }
  const int gq = Hq / Hkv;
  const long long items = (long long)n_tiles * Hkv * ((gq + 1) / 2);
  dim3 grid((unsigned)(items < sms ? items : sms));
  fz_launch(attn_prefill_pair_kernel<HD, BOX>, grid, dim3(PAIR_THREADS), smem, stream, qm, kvm, seg, tiles, n_tiles, table, mb,
            page_size, (__nv_bfloat16*)out, Hq, Hkv, scale * 1.4426950408889634f, window, part_o, part_ml, err);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

template <int HD, int BOX>
int launch(const void* q, int N, const void* k_pool, long long pool_rows, const int* seg, const int* tiles, int n_tiles,
           const int* table, int mb, int page_size, void* out, int Hq, int Hkv, float scale, int window, float* part_o,
           float* part_ml, int* err, cudaStream_t stream) {
  CUtensorMap qm, kvm;
  int st = get_map_bf16(q, N, Hq * HD, BM, &qm);
  if (st != FZ_OK) return st;
  if ((st = get_map_bf16(k_pool, pool_rows, HD, BOX, &kvm)) != FZ_OK) return st;
  constexpr int HALVES = HD / 64, HALF_BYTES = 128 * 128;
  constexpr int KV_STAGES = HD <= 64 ? 4 : 3;
  constexpr size_t smem = (size_t)HALVES * HALF_BYTES + KV_STAGES * 2 * HALVES * HALF_BYTES + 2 * BM * 4 + 8 * 32 + 1024;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  static bool raised = false;
  if (!raised) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<HD, BOX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    raised = true;
  }
  // one block per SM at most; each walks its share of the (tile, head) items
  const long long items = (long long)n_tiles * Hq;
  dim3 grid((unsigned)(items < sms ? items : sms));
  fz_launch(attn_prefill_tc_kernel<HD, BOX>, grid, dim3(NUM_THREADS), smem, stream, qm, kvm, seg, tiles, n_tiles, table, mb, page_size,
            (__nv_bfloat16*)out, Hq, Hkv, scale * 1.4426950408889634f, window, part_o, part_ml, err);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}
// Finishes the query tiles that were cut along the keys. splits: int32 [n_split][2] = (first entry, entries) of a tile,
// whose entries stand one after the other in the list. One warp per row (grid: 32 groups of four rows, heads, tiles),
// a lane owns HD / 32 neighbouring dimensions: the pieces' maxima first, then the pieces in entry order, each weighted
// by 2^(its maximum - the row's), and one division.
template <int HD>
__global__ void __launch_bounds__(128)
attn_prefill_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const int* __restrict__ seg,
                          const int* __restrict__ tiles, const int* __restrict__ splits, __nv_bfloat16* __restrict__ out, int Hq) {
  constexpr int PER = HD / 32;
  fz_grid_launch_dependents();
  fz_grid_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * 4 + warp, h = blockIdx.y;
  const int first = splits[2 * blockIdx.z], cnt = splits[2 * blockIdx.z + 1];
  const int s_idx = tiles[3 * first], r_off = tiles[3 * first + 1];
  if (s_idx < 0 || cnt <= 0) return;
  const int n_rows = seg[4 * s_idx + 1];
  if (r >= min(BM, n_rows - r_off)) return;
  const size_t row = (size_t)seg[4 * s_idx] + r_off + r;
  auto slot_row = [&](int e) { return ((size_t)(first + e) * Hq + h) * BM + r; };
  float M = -INFINITY;
  for (int e = lane; e < cnt; e += 32) M = fmaxf(M, part_ml[slot_row(e) * 2]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
  float acc[PER], l = 0.f;
#pragma unroll
  for (int j = 0; j < PER; ++j) acc[j] = 0.f;
  for (int e = 0; e < cnt; ++e) {
    const size_t sr = slot_row(e);
    const float2 ml = *(const float2*)(part_ml + sr * 2);
    const float f = ml.x == -INFINITY ? 0.f : exp2f(ml.x - M);      // a piece in which the row saw no key weighs nothing
    if (f == 0.f) continue;
    l += ml.y * f;
    const float* src = part_o + sr * HD + lane * PER;
#pragma unroll
    for (int j = 0; j < PER; ++j) acc[j] += src[j] * f;
  }
  const float inv = l > 0.f ? 1.0f / l : 0.f;
  __nv_bfloat16* dst = out + row * Hq * HD + (size_t)h * HD + lane * PER;
#pragma unroll
  for (int j = 0; j < PER; j += 2) {
    const __nv_bfloat162 pk = __floats2bfloat162_rn(acc[j] * inv, acc[j + 1] * inv);
    *(__nv_bfloat162*)(dst + j) = pk;
  }
}
}  // namespace

static int g_prefill_mode = 0;
// 0: choose by shape (the default); 1: always one head per block; 2: always two heads per block
FZ_API int fz_attn_prefill_tc_mode(int mode) {
  if (mode < 0 || mode > 2) return FZ_BAD_SHAPE;
  g_prefill_mode = mode;
  return FZ_OK;
}

// Takes head sizes 64 and 128 and page sizes 8, 16 and multiples of 16, with the pool laid out as (pages, 2, Hkv,
// page_size, hd); anything else is refused and the mma.sync kernel runs instead.
FZ_API int fz_attn_prefill_tc_check(int Hq, int Hkv, int hd, int page_size) {
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv) return FZ_BAD_SHAPE;
  if (hd != 64 && hd != 128) return FZ_BAD_SHAPE;
  if (!(page_size == 8 || (page_size > 0 && page_size % 16 == 0))) return FZ_BAD_SHAPE;
  return FZ_OK;
}

#ifdef FZ_ATTN_PROF
FZ_API int fz_attn_prefill_prof(unsigned long long* host32) {
  cudaError_t e = cudaMemcpyFromSymbol(host32, fz_attn_prof, sizeof(unsigned long long) * 32);
  unsigned long long zero[32] = {};
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(fz_attn_prof, zero, sizeof zero);
  return (int)e;
}
#endif
// tiles: int32 [n_tiles][3] = (portion index or -1, first row of the 128-row tile within the portion, range of key tiles or
// -1: see `entry_range`). q: [N, Hq * hd]. splits: int32 [n_split][2] = (first entry, entries) of every query tile that
// is cut along the keys; part_o / part_ml: float32 scratch of n_tiles * Hq * 128 * hd and n_tiles * Hq * 128 * 2 elements
// (only the slots of cut tiles are used; both may be null when n_split is 0).
FZ_API int fz_attn_prefill_tc(const void* q, int N, const void* k_pool, const void* v_pool, long long page_stride,
                              int num_pages, const int* seg, const int* tiles, int n_tiles, const int* splits, int n_split,
                              float* part_o, float* part_ml, const int* table, int mb, int page_size, void* out, int Hq,
                              int Hkv, int hd, float scale, int window, int* err, cudaStream_t stream) {
  if (n_tiles <= 0) return FZ_OK;
  if (fz_attn_prefill_tc_check(Hq, Hkv, hd, page_size) != FZ_OK || Hq > 65535) return FZ_BAD_SHAPE;
  if (n_split < 0 || (n_split > 0 && (!splits || !part_o || !part_ml))) return FZ_BAD_SHAPE;
  if (page_stride != 2LL * Hkv * page_size * hd ||
      (const __nv_bfloat16*)v_pool != (const __nv_bfloat16*)k_pool + (long long)Hkv * page_size * hd)
    return FZ_BAD_SHAPE;
  if ((((uintptr_t)q) | ((uintptr_t)k_pool) | ((uintptr_t)out) | ((uintptr_t)part_o) | ((uintptr_t)part_ml)) & 15) return FZ_BAD_ALIGNMENT;
  const long long pool_rows = (long long)num_pages * 2 * Hkv * page_size;
  // Which kernel: two heads per block where that fills the SMs (measured on a B200: it wins from about 1.5 items per SM
  // on at head size 128: 175 against 198 us for a 4,096-token portion of 32 / 8 heads, 8.4 against 10.1 ms for 32,768
  // tokens; with fewer items its coarser items balance worse, and at head size 64 it does not pay), else one head per
  // block. `fz_attn_prefill_tc_mode` overrides the choice (tests run both kernels on the same inputs).
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  const long long pair_items = (long long)n_tiles * Hkv * ((Hq / Hkv + 1) / 2);
  const bool single = g_prefill_mode == 1 || (g_prefill_mode == 0 && (hd != 128 || 2 * pair_items < 3LL * sms));
  int st = FZ_OK;
#define FZ_T(HD_, BOX_)                                                                                                          \
  st = single ? launch<HD_, BOX_>(q, N, k_pool, pool_rows, seg, tiles, n_tiles, table, mb, page_size, out, Hq, Hkv, scale,       \
                                  window, part_o, part_ml, err, stream)                                                          \
              : launch_pair<HD_, BOX_>(q, N, k_pool, pool_rows, seg, tiles, n_tiles, table, mb, page_size, out, Hq, Hkv,         \
                                       scale, window, part_o, part_ml, err, stream)
  // the largest box a page allows: a key tile of 128 keys is then 2, 8 or 16 boxes per column half
  if (hd == 64 && page_size == 8) FZ_T(64, 8);
  else if (hd == 64 && page_size % 64 == 0) FZ_T(64, 64);
  else if (hd == 64) FZ_T(64, 16);
  else if (page_size == 8) FZ_T(128, 8);
  else if (page_size % 64 == 0) FZ_T(128, 64);
  else FZ_T(128, 16);
#undef FZ_T
  if (st != FZ_OK || n_split == 0) return st;
  const dim3 grid(BM / 4, (unsigned)Hq, (unsigned)n_split);
  if (hd == 64) fz_launch(attn_prefill_merge_kernel<64>, grid, dim3(128), 0, stream, (const float*)part_o, (const float*)part_ml, seg, tiles, splits, (__nv_bfloat16*)out, Hq);
  else fz_launch(attn_prefill_merge_kernel<128>, grid, dim3(128), 0, stream, (const float*)part_o, (const float*)part_ml, seg, tiles, splits, (__nv_bfloat16*)out, Hq);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

#ifdef FZ_TIMELINE
FZ_TIMELINE_READER(attn_prefill_tc)
#endif
