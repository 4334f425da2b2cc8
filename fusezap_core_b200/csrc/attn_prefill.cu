// Causal flash attention for prompt portions over the paged bf16 cache, on tensor cores.
//
// grid (tiles, query heads, 2), 128 threads. The host lists tiles of 128 consecutive token rows of one portion (the ones
// with the most keys first); a CTA serves one 64-row half of a tile, warp w owns rows 16 w .. 16 w + 15 of it. The keys of the portion's request,
// from the start of the window (or 0) to the tile's last row's own position, come from the pages in tiles of 64
// through a two-stage cp.async ring; S = Q K^T and O += P V run on mma.sync m16n8k16 with float32 accumulators,
// softmax is online in the exp2 domain with float32 max and sum, and P is rounded to bf16 for the second product (as
// the reference's prefill kernel does: fusezap/device/cuda_kernels/attention.py:86-117, 255-326). The keys of this
// very step were written to the pages by the rotation kernel before, so a portion reads its own earlier rows from there.
// Key tiles start at multiples of 64 in absolute position, so a row's sums do not depend on how the prompt was cut.
#include "attn_mma.cuh"
#include <math.h>

namespace {
using namespace fzattn;

constexpr int BM = 64, BN = 64, THREADS = 128;

template <int HD>
__global__ void __launch_bounds__(THREADS)
attn_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                    const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ seg,
                    const int* __restrict__ tiles, const int* __restrict__ table, int mb, long long page_stride,
                    int page_size, __nv_bfloat16* __restrict__ out, int Hq, int Hkv, float scale_log2, int window) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  constexpr int KSTEPS = HD / 16, NB = HD / 8, TILE_BYTES = BN * HD * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t s_base = smem_u32(smem);          // [2 stages][K | V], then Q
  const uint32_t s_q = s_base + 4 * TILE_BYTES;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // the host lists 128-row tiles; blockIdx.z picks the 64-row half this CTA serves
  const int s_idx = tiles[3 * blockIdx.x], r_off = tiles[3 * blockIdx.x + 1] + BM * (int)blockIdx.z;
  if (s_idx < 0) return;
  const int h = blockIdx.y, kvh = h / (Hq / Hkv);
  const int row0 = seg[4 * s_idx], n_rows = seg[4 * s_idx + 1], pos0 = seg[4 * s_idx + 2];
  if (r_off >= n_rows) return;
  const int valid_rows = min(BM, n_rows - r_off);
  const int qpos0 = pos0 + r_off;                               // position of the tile's first row
  const int last_pos = qpos0 + valid_rows - 1;
  const int lo_tile = window > 0 ? max(0, qpos0 - window + 1) : 0;
  const int k_begin = lo_tile & ~(BN - 1);
  const int ntiles = (last_pos - k_begin) / BN + 1;
  const int* trow = table + (size_t)s_idx * mb;
  const long long head_off = (long long)kvh * page_size * HD;

  {
    const __nv_bfloat16* qbase = q + (size_t)(row0 + r_off) * Hq * HD + (size_t)h * HD;
    for (int e = tid; e < BM * (HD / 8); e += THREADS) {
      const int r = e / (HD / 8), c = e - r * (HD / 8);
      cp_async16(s_q + swz<HD>(r, c), qbase + (size_t)r * Hq * HD + c * 8, r < valid_rows);
    }
  }
  auto issue = [&](int t) {
    const uint32_t st = s_base + (t & 1) * 2 * TILE_BYTES;
    load_kv_tile<HD, BN, THREADS>(st, st + TILE_BYTES, k_pool, v_pool, trow, page_stride, head_off, page_size,
                                  k_begin + t * BN, lo_tile, last_pos, tid);
    cp_async_commit();
  };
  issue(0);

  uint32_t qf[KSTEPS][4];
  float o[NB][4];
#pragma unroll
  for (int i = 0; i < NB; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int r_lo = warp * 16 + (lane >> 2);                     // this thread's rows: r_lo and r_lo + 8
  const int qp[2] = {qpos0 + r_lo, qpos0 + r_lo + 8};
  const int warp_first = qpos0 + warp * 16, warp_last = min(warp_first + 15, last_pos);

  for (int t = 0; t < ntiles; ++t) {
    if (t + 1 < ntiles) { issue(t + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    if (t == 0) {
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks)
        ldmatrix_x4(qf[ks], s_q + swz<HD>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));
    }
    const int key0 = k_begin + t * BN;
    // a warp whose rows all lie before this key tile, or whose windows all ended before it, has nothing to do here
    const bool active = key0 <= warp_last && (window <= 0 || key0 + BN - 1 >= warp_first - window + 1) && warp * 16 < valid_rows;
    if (active) {
      const uint32_t sk = s_base + (t & 1) * 2 * TILE_BYTES, sv = sk + TILE_BYTES;
      float s[BN / 8][4];
#pragma unroll
      for (int j = 0; j < BN / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
        for (int jb = 0; jb < BN / 16; ++jb) {
          uint32_t kf[4];
          const int mi = lane >> 3;
          ldmatrix_x4(kf, sk + swz<HD>(jb * 16 + (mi >> 1) * 8 + (lane & 7), ks * 2 + (mi & 1)));
          mma_bf16(s[2 * jb], qf[ks], kf[0], kf[1]);
          mma_bf16(s[2 * jb + 1], qf[ks], kf[2], kf[3]);
        }
      }
      // mask: needed only where the tile touches the diagonal or the window's edge
      const bool need_mask = key0 + BN - 1 > warp_first || (window > 0 && key0 < warp_last - window + 1);
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < BN / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = s[j][e] * scale_log2;
          if (need_mask) {
            const int key = key0 + 8 * j + 2 * (lane & 3) + (e & 1);
            const int qpos = qp[e >> 1];
            const bool ok = key <= qpos && (window <= 0 || key >= qpos - window + 1);
            v = ok ? v : -INFINITY;
          }
          s[j][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      float corr[2], mu[2];
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 1));
        mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 2));
        const float mn = fmaxf(m_run[hh], mx[hh]);
        mu[hh] = mn == -INFINITY ? 0.f : mn;
        corr[hh] = exp2f(m_run[hh] - mu[hh]);
        m_run[hh] = mn;
      }
      float sum[2] = {0.f, 0.f};
#pragma unroll
      for (int j = 0; j < BN / 8; ++j) {
        s[j][0] = exp2f(s[j][0] - mu[0]); s[j][1] = exp2f(s[j][1] - mu[0]);
        s[j][2] = exp2f(s[j][2] - mu[1]); s[j][3] = exp2f(s[j][3] - mu[1]);
        sum[0] += s[j][0] + s[j][1];
        sum[1] += s[j][2] + s[j][3];
      }
      l_run[0] = l_run[0] * corr[0] + sum[0];
      l_run[1] = l_run[1] * corr[1] + sum[1];
#pragma unroll
      for (int i = 0; i < NB; ++i) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
#pragma unroll
      for (int kk = 0; kk < BN / 16; ++kk) {       // 16 keys per k-step
        uint32_t pf[4];
        pf[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        pf[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        pf[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        pf[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int nb = 0; nb < NB; nb += 2) {
          uint32_t vf[4];
          const int mi = lane >> 3;
          ldmatrix_x4_trans(vf, sv + swz<HD>(kk * 16 + (mi & 1) * 8 + (lane & 7), nb + (mi >> 1)));
          mma_bf16(o[nb], pf, vf[0], vf[1]);
          mma_bf16(o[nb + 1], pf, vf[2], vf[3]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 1);
    l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 2);
  }
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int r = r_lo + 8 * hh;
    if (r >= valid_rows) continue;
    const float inv = 1.0f / l_run[hh];
    __nv_bfloat16* orow = out + (size_t)(row0 + r_off + r) * Hq * HD + (size_t)h * HD + 2 * (lane & 3);
#pragma unroll
    for (int i = 0; i < NB; ++i)
      *(uint32_t*)(orow + 8 * i) = pack_bf16(o[i][2 * hh] * inv, o[i][2 * hh + 1] * inv);
  }
}

template <int HD>
int launch(const void* q, const void* k_pool, const void* v_pool, const int* seg, const int* tiles, int n_tiles,
           const int* table, int mb, long long page_stride, int page_size, void* out, int Hq, int Hkv, float scale,
           int window, cudaStream_t stream) {
  constexpr size_t smem = 4 * (BN * HD * 2) + BM * HD * 2;
  static bool raised = false;
  if (smem > 48 * 1024 && !raised) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    raised = true;
  }
  dim3 grid(n_tiles, Hq, 2);
  fz_launch(attn_prefill_kernel<HD>, grid, dim3(THREADS), smem, stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool,
            (const __nv_bfloat16*)v_pool, seg, tiles, table, mb, page_stride, page_size, (__nv_bfloat16*)out, Hq, Hkv,
            scale * 1.4426950408889634f, window);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}
}  // namespace

FZ_API int fz_attn_prefill_check(int Hq, int Hkv, int hd) {
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv) return FZ_BAD_SHAPE;
  if (hd != 64 && hd != 128) return FZ_BAD_SHAPE;
  return FZ_OK;
}

// tiles: int32 [n_tiles][3] = (segment index or -1, first row of the 128-row tile within the portion, -1: this kernel
// takes no tile that is cut along the keys).
FZ_API int fz_attn_prefill(const void* q, const void* k_pool, const void* v_pool, const int* seg, const int* tiles,
                           int n_tiles, const int* table, int mb, long long page_stride, int page_size, void* out,
                           int Hq, int Hkv, int hd, float scale, int window, cudaStream_t stream) {
  if (n_tiles <= 0) return FZ_OK;
  if (fz_attn_prefill_check(Hq, Hkv, hd) != FZ_OK || page_size <= 0 || Hq > 65535) return FZ_BAD_SHAPE;
  if (hd == 64)
    return launch<64>(q, k_pool, v_pool, seg, tiles, n_tiles, table, mb, page_stride, page_size, out, Hq, Hkv, scale, window, stream);
  return launch<128>(q, k_pool, v_pool, seg, tiles, n_tiles, table, mb, page_stride, page_size, out, Hq, Hkv, scale, window, stream);
}

#ifdef FZ_TIMELINE
FZ_TIMELINE_READER(attn_prefill)
#endif
